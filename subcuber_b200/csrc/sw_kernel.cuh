// Persistent, warp-specialised tile-program GEMM kernel for sm_100a.
//
// One CTA per SM walks a static list of output tiles.  For every tile it interprets a tile program
// (tile_program.h): a sequence of half-size products (level 1: the seven Strassen-Winograd products of
// src/algos/strassen_winograd_level1.py:16-42 in the reference project; level 0: one product) and a
// sequence of epilogue steps that apply the postsums and write C.  It replaces, for this path, the
// reference's per-CTA kernel (include/cutlass/gemm/kernel/strassen_gemm.h:419-1460), its multistage
// mainloop with presum (gemm/threadblock/strassen_mma_multistage.h), its postsum epilogues
// (epilogue/threadblock/strassen_epilogue.h, strassen_interim_epilogue.h) and the cross-kernel
// PostsumSemaphore: products that feed one output tile run back to back in ONE CTA and hand their
// accumulators over inside tensor memory, so no cross-CTA flag exists.
//
// Warp roles (one CTA = 6 or 10 warps):
//   warp 0      TMA producer: non-multicast tiled bulk loads of single-term operands into the stage ring
//   warp 1      MMA issuer: tcgen05.mma (kind::f16 or kind::tf32, fp32 accumulators in TMEM), one thread
//   warps 2-5   epilogue: tcgen05.ld -> registers -> postsum -> vectorised global stores
//   warps 6-7   two more TMA producers: the three take the k-steps in turn (loads of one warp complete one after
//               the other, about 240 ns apiece on B200 whatever their size; loads of different warps overlap)
//   warps 8-11  presum warps (modes FEED and JOB only)
//                 FEED: form multi-term operand tiles S/T = +-X +-Y ... in shared memory, in the swizzled
//                       layout the MMA reads, straight from the raw quadrant values (one rounding)
//                 JOB : materialise the eight presums into a global workspace while the MMA pipeline of the
//                       same launch computes the products that need no presum (the reference's
//                       "interleaved presum", strassen_mma_multistage.h:1536-1726)
//
// Shared-memory stage (48 KiB at BN = 256): A tile 128 rows x 128 B (K-major, 128B swizzle) followed by the
// B tile as BN*ESIZE/128 blocks of [BK rows x 128 B] (N-major, 128B swizzle), exactly as TMA deposits them.
#pragma once
#include <cuda_bf16.h>

#include "ptx.cuh"
#include "tile_program.h"
#include "epilogue.cuh"

namespace sb200 {

enum PresumMode { kPresumNone = 0, kPresumFeed = 1, kPresumJob = 2 };

enum StatusCode {
  kStatusOk = 0,
  kStatusProducerTimeout = 101,
  kStatusMmaTimeout = 102,
  kStatusEpilogueTimeout = 103,
  kStatusPresumTimeout = 104,
  kStatusSplitTimeout = 105,
};

struct View {
  const void* ptr;  // first element of the view
  long long ld;     // leading dimension in elements
  int rows;         // extent of the slow dimension
  int cols;         // extent of the contiguous dimension
};

// One presum job: the four combinations of one operand's quadrants, written as four packed matrices.
//   side 0 (A): S1, S2, A02, A1S2      side 1 (B): B10, B31, S3, S3B2
//   npairs > 0: instead, `npairs` two-term combinations given by table, result r = c0 * quadrant q0 + c1 * quadrant q1
//               with pair_q[r] = {q0, q1}, pair_c[r] = {c0, c1} (coefficients +1 or -1): the presums of algorithms
//               whose operand sums have two terms (Strassen's original algorithm)
constexpr int SB200_MAX_PRESUM_PAIRS = 6;
struct PresumSideJob {
  const void* src[4];  // quadrant base pointers, row-major with a common leading dimension
  long long ld;        // in elements
  void* dst;           // [4 or npairs][rows][cols], packed
  int rows, cols;      // extent of one quadrant (and of each result)
  int rows2, cols2;    // rows present in quadrants 2, 3 and columns present in quadrants 1, 3 (<= rows, cols): an
                       // operand whose extents are not twice the block extents reads as if padded with zeros
  int side;
  int npairs;
  signed char pair_q[SB200_MAX_PRESUM_PAIRS][2];
  signed char pair_c[SB200_MAX_PRESUM_PAIRS][2];
};
constexpr int SB200_MAX_JOBS = 4;

// One-launch plan: the presum warps publish the presums panel by panel, and the TMA producers wait for the two panels
// a tile reads before its first product on presum operands.  A panel is the block of rows of the four A-side presums
// that one tile row reads (or the block of columns of the four B-side presums that one tile column reads); it is
// produced in `chunks` pieces along K, each by the presum warps of one CTA, drawn from a list that follows the tile
// raster: the A panels of the first band, every B panel, then the A panels of the other bands.
struct PresumPanels {
  int enabled;
  int chunks;        // pieces per panel; a panel is ready when its counter has reached this
  int chunk_k;       // extent of a piece along K, in elements
  int panel_rows;    // rows of an A panel (tile rows of a worker)
  int panel_cols;    // columns of a B panel
  int group_cols;    // tile columns in flight at once (workers / band, rounded up): see the producer's wait
  int* next_chunk;   // global counter over the chunk list (zero at launch)
  int* ready_a;      // [tiles_m] pieces finished per A panel (zero at launch)
  int* ready_b;      // [tiles_n]
};

struct KernelParams {
  CUtensorMap tmap[SB200_NUM_VIEWS];
  // CTA-pair kernels whose unit list has column halves, blocked B maps: the B-side views (SB200_VIEW_B0 ...) once
  // more with half as many column blocks per box, for the loads of a column half
  CUtensorMap tmap_half_b[SB200_NUM_VIEWS - SB200_VIEW_B0];
  View view[SB200_NUM_VIEWS];
  void* out[4];       // output quadrant base pointers (level 0: out[0] = D)
  long long ldo;      // leading dimension of the output in elements
  int bf16;           // 16-bit kernels only: the operand and output type is bfloat16 (else IEEE half)
  int out_rows;       // rows of one output quadrant
  int out_cols;       // columns of one output quadrant
  int out_rows2;      // rows present in output quadrants 2, 3 and columns present in quadrants 1, 3 (<= out_rows,
  int out_cols2;      //   out_cols): the rest of those blocks lies outside the output matrix and is not stored
  // output scaling: every value written to an output quadrant is alpha * sum + beta * C (cin[q] is null when beta = 0)
  float alpha, beta;
  const void* cin[4];
  long long ldc;
  float* ws[SB200_NUM_WS];  // fp32 hand-off buffers, tile-contiguous: [tile id][BN/32][128][32]
  int tiles_m, tiles_n;     // tile grid over one output quadrant
  int num_k;                // k-steps per product
  int band;                 // raster band height in tiles
  int b_blocked;            // 1: the B tensor maps are 3-D [128-byte column block][row][block]: one load per B tile
  // The unit list (see WorkUnit): whole_tiles whole tiles, then two units for each of the region_tiles tiles that
  // follow: its column halves (region_cols = 1) or its K-halves (region_cols = 0; the first half hands its partial
  // sums over through split_buf and raises split_flags).
  int whole_tiles;
  int region_tiles;
  int region_cols;
  int* unit_counter;        // CTA-pair kernels: units are drawn from this counter (zero at launch) in list order by
                            // whichever pair is free; null: dealt round-robin
  int split_epoch;          // value a raised flag holds in this launch (flags are zeroed once per run)
  float* split_buf;         // [split slot][quadrant 4][CTA of the tile][128 x BN] fp32, hand-off tile order
  int* split_flags;         // [split slot][quadrant 4][CTA of the tile 2][epilogue warp 4]
  int* status;              // device status word, 0 = ok
  unsigned long long wait_ns;  // bound of every wait in the kernel (mbarrier, split flag), in nanoseconds
  int drop_split_flags;     // test aid for the give-up path: first halves of split tiles do not raise their flags
#ifdef SB200_PROFILE
  int debug_flags;          // measurement aids (results are garbage): bit 0 = issue no MMA, bit 1 = issue no TMA load,
                            // bit 3 = load only while the ring fills for the first time (pairs), bit 4 = skip the
                            // presum job (pairs), bit 5 = skip the epilogue bodies
  long long* prof;          // measurement aid (CTA-pair kernels): 8 cycle counters per CTA, or null
  int hint_mode;            // measurement aid: L2 cache hints of the operand loads (pairs): tens digit = A, units = B;
                            // 0 none, 1 evict_first, 2 evict_last, 3 evict_normal
#endif
  PresumPanels panels;      // mode JOB, one-launch plan only
  // presum jobs (mode JOB), run by the presum warps of the whole grid one after the other
  int njobs;
  PresumSideJob job[SB200_MAX_JOBS];
  sb200_program_t prog;
};

// Measurement aids exist only in builds with -DSB200_PROFILE; the product kernels carry none of their branches.
#ifdef SB200_PROFILE
#define SB200_DEBUG_BIT(p, bit) (((p).debug_flags & (bit)) != 0)
#define SB200_PROF_PTR(p) ((p).prof)
#else
#define SB200_DEBUG_BIT(p, bit) false
#define SB200_PROF_PTR(p) (static_cast<long long*>(nullptr))
#endif

template <int ESIZE_, int BN_, int STAGES_, int MODE_, bool SCALED_ = false>
struct KernelConfig {
  static constexpr bool SCALED = SCALED_;  // D = alpha * sum + beta * C instead of D = sum
  static constexpr int ESIZE = ESIZE_;            // operand element size: 2 (f16) or 4 (f32 storage, tf32 math)
  static constexpr int BM = 128;
  static constexpr int BN = BN_;
  static constexpr int BK = 128 / ESIZE;          // elements per 128-byte swizzle row
  static constexpr int STAGES = STAGES_;
  static constexpr int MODE = MODE_;
  // fp32 sources an epilogue step may sum (hand-off tiles of the program, + one of the level above, + the partial
  // sum of a split tile).  The kernels with presum warps have a smaller register budget and run programs that
  // need fewer: JOB = first launch of the interleaved plan (1 + 1), FEED = one fused launch, never linked or split.
  static constexpr int NSRC_MAX = MODE_ == 0 ? SB200_MAX_SRC_TERMS + 1 : (MODE_ == 2 ? 2 : 1);
  // TMEM slots a step may sum: the programs of the kernels without presum warps read one slot per step
  static constexpr int NSLOT_MAX = MODE_ == 0 ? 1 : 2;
  static constexpr int UMMA_K = 32 / ESIZE;
  static constexpr int KSUB = BK / UMMA_K;        // MMAs per stage (4)
  static constexpr int A_BYTES = BM * 128;
  static constexpr int NBLK = BN * ESIZE / 128;   // 128-byte-wide column blocks of the B tile
  static constexpr int BLK_BYTES = BK * 128;
  static constexpr int B_BYTES = NBLK * BLK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SLOTS = 512 / BN;
  static constexpr int TMEM_COLS = 512;
  static constexpr int PRESUM_WARPS = (MODE == kPresumNone) ? 0 : 4;
  static constexpr int FIRST_PRESUM_WARP = 8;
  static constexpr int THREADS = (FIRST_PRESUM_WARP + PRESUM_WARPS) * 32;
  static constexpr int BAR_BYTES = 1024;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + kStagingBytes + 1024;  // +1024: manual alignment slack
  static constexpr uint32_t FMT = (ESIZE == 2) ? 0u : 2u;
  // B tile (N contiguous): 16-bit elements use the plain 128-byte swizzle with 8-row groups; 32-bit elements
  // must use the 128-byte swizzle with 32-byte atoms, whose pattern repeats every 4 rows.
  static constexpr bool B_SWZ32 = (ESIZE == 4);
  static constexpr uint32_t B_LAYOUT_TYPE = B_SWZ32 ? 1u : 2u;
  static constexpr uint32_t B_SBO = B_SWZ32 ? 512u : 1024u;
};

struct TileCoord {
  int i, j, id;
};

__device__ __forceinline__ TileCoord tile_of(int w, int tiles_m, int tiles_n, int band) {
  int per_band = band * tiles_n;
  int b = w / per_band;
  int r = w - b * per_band;
  int rows_in_band = min(band, tiles_m - b * band);
  TileCoord t;
  t.i = b * band + (r % rows_in_band);
  t.j = r / rows_in_band;
  t.id = t.i * tiles_n + t.j;
  return t;
}

// Work units of the persistent loop.  A unit is one output tile, one column half of a tile, or one K-half of a tile.
// Column halves (CTA-pair kernels): the two halves are independent units that run the tile program on 128 of the
// tile's 256 columns (MMA N = 128, half the B columns, half the epilogue chunks); a half has a whole unit's ratio of
// MMA work to epilogue work, and its results are bit-identical to the whole tile's.  The host cuts the tiles of a last
// wave that is at most half full into column halves, so that this wave lasts half as long.
// K-halves (1-CTA kernels, tiles dealt round-robin): every postsum is linear in
// the products, so both halves of a tile run the whole tile program on their K range with private hand-off tiles; at
// each step that leaves the tile (an output quadrant or a buffer of the level above) the first half (the publisher)
// writes its partial sum to a split buffer and raises a flag, and the second half (the finisher) waits (bounded) for
// the flag and adds the partial sum.  The unit list, in the order units are handed out:
//   units 0 .. whole_tiles - 1            whole tiles in raster order
//   then 2 units per tile of the region   first half, second half of tiles whole_tiles .. whole_tiles + region_tiles - 1
// The host cuts the tiles of a last wave that is at most half full when tiles are dealt round-robin: that wave then
// lasts half as long.  Both halves of a tile start at the same time on two workers,
// at the same phase as every other half: workers that share operand panels stay close in K, which is what lets them
// share those panels through L2.  (Cutting tiles at uneven points to give every worker an exactly equal share of a
// partial wave was tried and is much slower: workers at different K phases stop sharing panels and the launch
// becomes memory bound.)
struct WorkUnit {
  int tile;       // linear tile index (argument of tile_of)
  int part;       // 0 = whole tile or publisher, 1 = finisher
  int nparts;     // 1 or 2
  int k0, k1;     // k-step range [k0, k1)
  int ws_slot;    // tile slot of this unit in the level-1 hand-off buffers (a finisher uses an extra slot)
  int split_idx;  // slot of the cut tile in the split buffer and the flag array
  int col_part;   // column half of the tile this unit computes (0 when the tile's columns are not cut)
  int col_parts;  // 1 = all columns of the tile, 2 = one half
};

__host__ __device__ __forceinline__ int total_units(const KernelParams& p) { return p.whole_tiles + 2 * p.region_tiles; }

// Unit number `u` of the list.
__host__ __device__ __forceinline__ WorkUnit unit_of(const KernelParams& p, int u) {
  WorkUnit w;
  w.col_part = 0; w.col_parts = 1;
  if (u < p.whole_tiles) {
    w.tile = u; w.part = 0; w.nparts = 1; w.k0 = 0; w.k1 = p.num_k; w.ws_slot = u; w.split_idx = 0;
  } else if (p.region_cols) {
    const int v = u - p.whole_tiles;
    w.tile = p.whole_tiles + (v >> 1);
    w.part = 0; w.nparts = 1; w.k0 = 0; w.k1 = p.num_k; w.ws_slot = w.tile; w.split_idx = 0;
    w.col_part = v & 1; w.col_parts = 2;
  } else {
    const int v = u - p.whole_tiles;
    const int h = p.num_k >> 1;
    w.split_idx = v >> 1;
    w.tile = p.whole_tiles + w.split_idx;
    w.part = v & 1;
    w.nparts = 2;
    w.k0 = w.part ? h : 0;
    w.k1 = w.part ? p.num_k : h;
    w.ws_slot = w.part ? p.tiles_m * p.tiles_n + w.split_idx : w.tile;
  }
  return w;
}

// The first code to arrive stays in the status word.  The code is published before the CTA-wide abort flag, so that
// roles which give up only because they saw the flag cannot overwrite the code of the wait that actually ran out.
__device__ __forceinline__ void raise_abort(const KernelParams& p, volatile int* abort_flag, int code) {
  const int before = atomicCAS(p.status, 0, code);
  __threadfence();
  *abort_flag = before == 0 ? 1 : 2;  // the store depends on the atomic's result, so it cannot pass it
}

// ---------------------------------------------------------------------------------------------------
// Presum arithmetic on one 16-byte vector per term.  Terms are combined left to right in fp32 (fp16
// operands) or fp32 (f32 operands) and rounded once, which is the reference oracle's convention
// (src/cuda/strassen_reference_l1.cuh:68-85).
template <int ESIZE>
struct VecAcc;

template <>
struct VecAcc<2> {
  float v[8];
  bool bf;  // the 16-bit type is bfloat16 (else IEEE half)
  __device__ __forceinline__ explicit VecAcc(bool is_bf16) : bf(is_bf16) {}
  __device__ __forceinline__ float2 widen(uint32_t pair) const {
    if (bf) return make_float2(__uint_as_float(pair << 16), __uint_as_float(pair & 0xffff0000u));
    return __half22float2(*reinterpret_cast<const __half2*>(&pair));
  }
  __device__ __forceinline__ void set(uint4 x, int c) {
    const uint32_t* h = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 f = widen(h[q]);
      v[2 * q] = c > 0 ? f.x : -f.x;
      v[2 * q + 1] = c > 0 ? f.y : -f.y;
    }
  }
  __device__ __forceinline__ void add(uint4 x, int c) {
    const uint32_t* h = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 f = widen(h[q]);
      v[2 * q] = c > 0 ? __fadd_rn(v[2 * q], f.x) : __fsub_rn(v[2 * q], f.x);
      v[2 * q + 1] = c > 0 ? __fadd_rn(v[2 * q + 1], f.y) : __fsub_rn(v[2 * q + 1], f.y);
    }
  }
  __device__ __forceinline__ uint4 pack() const {
    uint4 o;
    if (bf) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
    } else {
      __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) h[q] = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
    }
    return o;
  }
};

template <>
struct VecAcc<4> {
  float v[4];
  __device__ __forceinline__ explicit VecAcc(bool) {}
  __device__ __forceinline__ void set(uint4 x, int c) {
    const float* f = reinterpret_cast<const float*>(&x);
#pragma unroll
    for (int q = 0; q < 4; ++q) v[q] = c > 0 ? f[q] : -f[q];
  }
  __device__ __forceinline__ void add(uint4 x, int c) {
    const float* f = reinterpret_cast<const float*>(&x);
#pragma unroll
    for (int q = 0; q < 4; ++q) v[q] = c > 0 ? __fadd_rn(v[q], f[q]) : __fsub_rn(v[q], f[q]);
  }
  __device__ __forceinline__ uint4 pack() const {
    uint4 o;
    float* f = reinterpret_cast<float*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) f[q] = v[q];
    return o;
  }
};

// Combine the terms of `op` for the tile whose slow-dimension origin is `row0` and whose contiguous-dimension
// origin is `col0` (both in elements of the operand views) and write it into the stage buffer.
//   ROWS          rows of the tile in shared memory (A: 128 tile rows; B: BK k-rows)
//   VEC_PER_ROW   16-byte vectors per tile row (A: 8; B: BN*ESIZE/16)
//   block stride  bytes between 128-byte-wide column blocks (A: unused; B: BK*128)
//   SWZ32         false: 16-byte chunk index XOR (row & 7); true: 32-byte chunk index XOR (row & 3)
template <int ESIZE, int ROWS, int VEC_PER_ROW, int NTHREADS, bool SWZ32>
__device__ __forceinline__ void build_operand_tile(uint32_t smem_tile, uint32_t blk_bytes, const sb200_operand_t& op,
                                                   const View* views, int row0, int col0, int tid, bool bf) {
  constexpr int EPV = 16 / ESIZE;  // elements per vector
  constexpr int TOTAL = ROWS * VEC_PER_ROW;
  const int nterms = op.nterms;
#pragma unroll 2
  for (int v = tid; v < TOTAL; v += NTHREADS) {
    int r = v / VEC_PER_ROW;
    int cv = v - r * VEC_PER_ROW;
    int grow = row0 + r;
    int gcol = col0 + cv * EPV;
    uint4 x[SB200_MAX_TERMS];
#pragma unroll
    for (int t = 0; t < SB200_MAX_TERMS; ++t) {
      x[t] = make_uint4(0u, 0u, 0u, 0u);
      if (t < nterms) {
        const View& vw = views[op.view[t]];
        if (grow < vw.rows && gcol < vw.cols) {
          const char* src = static_cast<const char*>(vw.ptr) + (static_cast<long long>(grow) * vw.ld + gcol) * ESIZE;
          x[t] = ptx::ldg_nc_v4(src);
        }
      }
    }
    VecAcc<ESIZE> acc(bf);
    acc.set(x[0], op.coef[0]);
#pragma unroll
    for (int t = 1; t < SB200_MAX_TERMS; ++t)
      if (t < nterms) acc.add(x[t], op.coef[t]);
    int blk = cv >> 3;
    int ch = cv & 7;
    const int sch = SWZ32 ? ((((ch >> 1) ^ (r & 3)) << 1) | (ch & 1)) : (ch ^ (r & 7));
    uint32_t dst = smem_tile + blk * blk_bytes + r * 128 + (sch << 4);
    ptx::sts_v4(dst, acc.pack());
  }
}

// Global presum jobs: every presum thread of the grid takes 16-byte vector positions of a quadrant in a grid-stride
// loop; per position it reads the four raw quadrant vectors and writes the four combinations of that side.
// Sums are formed from the raw values left to right in fp32 and rounded once (VecAcc).
// `presum_rect` does this for the rectangle [row0, row1) x [col0, col1) of the quadrant (columns on 16-byte vectors).
template <int ESIZE>
__device__ __forceinline__ void presum_rect(const PresumSideJob& j, int row0, int row1, int col0, int col1, int gtid,
                                            int gthreads, bool bf) {
  constexpr int EPV = 16 / ESIZE;
  constexpr int U = 4;  // vector positions per thread per iteration: 16 loads in flight hide the memory latency
  const int vec_per_row = (col1 - col0) / EPV;
  const long long total = static_cast<long long>(row1 - row0) * vec_per_row;
  const long long q = static_cast<long long>(j.rows) * j.cols * ESIZE;  // bytes per result matrix
  const char* s0 = static_cast<const char*>(j.src[0]);
  const char* s1 = static_cast<const char*>(j.src[1]);
  const char* s2 = static_cast<const char*>(j.src[2]);
  const char* s3 = static_cast<const char*>(j.src[3]);
  char* out = static_cast<char*>(j.dst);
  for (long long v0 = gtid; v0 < total; v0 += static_cast<long long>(gthreads) * U) {
    uint4 x0[U], x1[U], x2[U], x3[U];
    long long o[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + static_cast<long long>(u) * gthreads;
      o[u] = -1;
      if (v < total) {
        const int rr = static_cast<int>(v / vec_per_row);
        const int r = row0 + rr;
        const int c = col0 + static_cast<int>(v - static_cast<long long>(rr) * vec_per_row) * EPV;
        const long long in = (r * j.ld + c) * ESIZE;
        const bool has_r = r < j.rows2, has_c = c < j.cols2;
        const uint4 zero = make_uint4(0, 0, 0, 0);
        x0[u] = ptx::ldg_nc_v4(s0 + in);
        x1[u] = has_c ? ptx::ldg_nc_v4(s1 + in) : zero;
        x2[u] = has_r ? ptx::ldg_nc_v4(s2 + in) : zero;
        x3[u] = (has_r && has_c) ? ptx::ldg_nc_v4(s3 + in) : zero;
        o[u] = (static_cast<long long>(r) * j.cols + c) * ESIZE;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (o[u] < 0) continue;
      if (j.side == 0) {
        // A side: S1 = A2 + A3, S2 = S1 - A0, A02 = A0 - A2, A1S2 = A1 - S2
        VecAcc<ESIZE> s(bf);
        s.set(x2[u], 1); s.add(x3[u], 1);                             // S1
        *reinterpret_cast<uint4*>(out + 0 * q + o[u]) = s.pack();
        s.add(x0[u], -1);                                             // S2 = S1 - A0 (unrounded S1)
        *reinterpret_cast<uint4*>(out + 1 * q + o[u]) = s.pack();
        VecAcc<ESIZE> t(bf);
        t.set(x0[u], 1); t.add(x2[u], -1);                            // A02
        *reinterpret_cast<uint4*>(out + 2 * q + o[u]) = t.pack();
        VecAcc<ESIZE> w(bf);                                              // A1S2 = A1 - S2 with the unrounded S2
        w.set(x2[u], -1); w.add(x3[u], -1); w.add(x0[u], 1); w.add(x1[u], 1);
        *reinterpret_cast<uint4*>(out + 3 * q + o[u]) = w.pack();
      } else {
        // B side: B10 = B1 - B0, B31 = B3 - B1, S3 = B31 + B0, S3B2 = S3 - B2
        VecAcc<ESIZE> s(bf);
        s.set(x1[u], 1); s.add(x0[u], -1);                            // B10
        *reinterpret_cast<uint4*>(out + 0 * q + o[u]) = s.pack();
        VecAcc<ESIZE> t(bf);
        t.set(x3[u], 1); t.add(x1[u], -1);                            // B31
        *reinterpret_cast<uint4*>(out + 1 * q + o[u]) = t.pack();
        t.add(x0[u], 1);                                              // S3 = B31 + B0 (unrounded B31)
        *reinterpret_cast<uint4*>(out + 2 * q + o[u]) = t.pack();
        t.add(x2[u], -1);                                             // S3B2 = S3 - B2 (unrounded S3)
        *reinterpret_cast<uint4*>(out + 3 * q + o[u]) = t.pack();
      }
    }
  }
}

// Table-driven two-term presums over a whole quadrant (PresumSideJob::npairs > 0): result r = c0 * quadrant q0 +
// c1 * quadrant q1, fp32 sum of the raw values, one rounding.  A function of its own, so that the loop above stays
// as it is for the plans that run beside products.
template <int ESIZE>
__device__ __forceinline__ void presum_pairs(const PresumSideJob& j, int gtid, int gthreads, bool bf) {
  constexpr int EPV = 16 / ESIZE;
  constexpr int U = 4;
  const int vec_per_row = j.cols / EPV;
  const long long total = static_cast<long long>(j.rows) * vec_per_row;
  const long long q = static_cast<long long>(j.rows) * j.cols * ESIZE;  // bytes per result matrix
  char* out = static_cast<char*>(j.dst);
  for (long long v0 = gtid; v0 < total; v0 += static_cast<long long>(gthreads) * U) {
    uint4 x[U][4];
    long long o[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + static_cast<long long>(u) * gthreads;
      o[u] = -1;
      if (v < total) {
        const int r = static_cast<int>(v / vec_per_row);
        const int c = static_cast<int>(v - static_cast<long long>(r) * vec_per_row) * EPV;
        const long long in = (r * j.ld + c) * ESIZE;
        const bool has_r = r < j.rows2, has_c = c < j.cols2;
        const uint4 zero = make_uint4(0, 0, 0, 0);
        x[u][0] = ptx::ldg_nc_v4(static_cast<const char*>(j.src[0]) + in);
        x[u][1] = has_c ? ptx::ldg_nc_v4(static_cast<const char*>(j.src[1]) + in) : zero;
        x[u][2] = has_r ? ptx::ldg_nc_v4(static_cast<const char*>(j.src[2]) + in) : zero;
        x[u][3] = (has_r && has_c) ? ptx::ldg_nc_v4(static_cast<const char*>(j.src[3]) + in) : zero;
        o[u] = (static_cast<long long>(r) * j.cols + c) * ESIZE;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (o[u] < 0) continue;
      for (int r = 0; r < j.npairs; ++r) {
        const int q0 = j.pair_q[r][0], q1 = j.pair_q[r][1];
        const uint4 y0 = q0 == 0 ? x[u][0] : (q0 == 1 ? x[u][1] : (q0 == 2 ? x[u][2] : x[u][3]));
        const uint4 y1 = q1 == 0 ? x[u][0] : (q1 == 1 ? x[u][1] : (q1 == 2 ? x[u][2] : x[u][3]));
        VecAcc<ESIZE> s(bf);
        s.set(y0, j.pair_c[r][0]);
        s.add(y1, j.pair_c[r][1]);
        *reinterpret_cast<uint4*>(out + r * q + o[u]) = s.pack();
      }
    }
  }
}

template <int ESIZE>
__device__ __forceinline__ void presum_side_job(const PresumSideJob& j, int gtid, int gthreads, bool bf) {
  if (j.npairs > 0) presum_pairs<ESIZE>(j, gtid, gthreads, bf);
  else presum_rect<ESIZE>(j, 0, j.rows, 0, j.cols, gtid, gthreads, bf);
}

// One-launch plan: the presum warps of a CTA (PT threads, `ptid` among them) draw chunks until the list is exhausted.
// `slot` is a word of shared memory for handing the drawn chunk number to the other presum threads; the two named
// barriers (ids 1 and 2) are used by the presum warps only.
template <int ESIZE, int PT>
__device__ __forceinline__ void presum_panels_job(const KernelParams& p, int ptid, volatile int* slot) {
  const PresumPanels& pp = p.panels;
  const int band0 = p.band < p.tiles_m ? p.band : p.tiles_m;   // A panels of the first raster band come first
  const int total = (p.tiles_m + p.tiles_n) * pp.chunks;
  const PresumSideJob& ja = p.job[0];
  const PresumSideJob& jb = p.job[1];
  while (true) {
    if (ptid == 0) *slot = atomicAdd(pp.next_chunk, 1);
    asm volatile("bar.sync 1, %0;" ::"r"(PT) : "memory");
    const int c = *slot;
    asm volatile("bar.sync 2, %0;" ::"r"(PT) : "memory");
    if (c >= total) break;
    int side, panel;
    const int piece = c % pp.chunks;
    const int q = c / pp.chunks;
    if (q < band0) { side = 0; panel = q; }
    else if (q < band0 + p.tiles_n) { side = 1; panel = q - band0; }
    else { side = 0; panel = q - p.tiles_n; }
    const int k0 = piece * pp.chunk_k;
    if (side == 0) {
      const int r0 = panel * pp.panel_rows;
      const int r1 = r0 + pp.panel_rows < ja.rows ? r0 + pp.panel_rows : ja.rows;
      const int k1 = k0 + pp.chunk_k < ja.cols ? k0 + pp.chunk_k : ja.cols;
      if (r0 < r1 && k0 < k1) presum_rect<ESIZE>(ja, r0, r1, k0, k1, ptid, PT, p.bf16 != 0);
    } else {
      const int c0 = panel * pp.panel_cols;
      const int c1 = c0 + pp.panel_cols < jb.cols ? c0 + pp.panel_cols : jb.cols;
      const int k1 = k0 + pp.chunk_k < jb.rows ? k0 + pp.chunk_k : jb.rows;
      if (c0 < c1 && k0 < k1) presum_rect<ESIZE>(jb, k0, k1, c0, c1, ptid, PT, p.bf16 != 0);
    }
    // every thread's stores are made visible device-wide (to TMA readers too), then one thread counts the piece
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"r"(PT) : "memory");
    if (ptid == 0) atomicAdd(side == 0 ? pp.ready_a + panel : pp.ready_b + panel, 1);
  }
}

// Bounded wait of a whole warp until the counter at `ctr` has reached `target`.
__device__ __forceinline__ bool wait_counter(const int* ctr, int target, volatile int* abort_flag, uint64_t limit_ns) {
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t polls = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (__all_sync(0xffffffffu, v >= target)) return true;
    if ((++polls & 63u) == 0) {
      const bool give_up = *abort_flag != 0 || ptx::globaltimer_ns() - t0 > limit_ns;
      if (__any_sync(0xffffffffu, give_up)) return false;
    }
    __nanosleep(100);
  }
}

template <int ESIZE>
__device__ __forceinline__ void presum_job(const KernelParams& p, int gtid, int gthreads) {
  for (int j = 0; j < p.njobs; ++j) presum_side_job<ESIZE>(p.job[j], gtid, gthreads, p.bf16 != 0);
}

// ---------------------------------------------------------------------------------------------------
template <typename Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1) sw_tile_program_kernel(const __grid_constant__ KernelParams p) {
  constexpr int ESIZE = Cfg::ESIZE;
  constexpr int BN = Cfg::BN;
  constexpr int BK = Cfg::BK;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int SLOTS = Cfg::SLOTS;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_base = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* slot_full = empty_bar + STAGES;
  uint64_t* slot_free = slot_full + SLOTS;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(slot_free + SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const uint32_t staging = ptx::smem_u32(bar_base + Cfg::BAR_BYTES);  // epilogue staging rows (epilogue.cuh)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_units = total_units(p);  // tiles, or K-halves of tiles, dealt round-robin
  const int nproducts = p.prog.nproducts;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1 + (Cfg::MODE == kPresumFeed ? Cfg::PRESUM_WARPS : 0));
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < SLOTS; ++s) {
      ptx::mbar_init(&slot_full[s], 1);
      ptx::mbar_init(&slot_free[s], 4);
    }
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0 || (warp >= 6 && warp < Cfg::FIRST_PRESUM_WARP)) {
    // ------------------------------------------------------------------ TMA producers (take the k-steps in turn)
    // Each producer warp runs its loop warp-uniformly and one elected lane issues (see ptx::elect_one).
    {
      const uint32_t my_turn = (warp == 0) ? 0u : static_cast<uint32_t>(warp - 5);
      uint32_t turn = 0;
      if (warp == 0 && lane == 0)
        for (int v = 0; v < SB200_NUM_VIEWS; ++v) ptx::prefetch_tmap(&p.tmap[v]);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; ok && u < num_units; u += gridDim.x) {
        const WorkUnit wu = unit_of(p, u);
        const TileCoord tile = tile_of(wu.tile, p.tiles_m, p.tiles_n, p.band);
        for (int ps = 0; ok && ps < nproducts; ++ps) {
          const sb200_product_t& pr = p.prog.product[ps];
          const bool a_tma = pr.a.nterms == 1;
          const bool b_tma = pr.b.nterms == 1;
          const uint32_t tx = (a_tma ? Cfg::A_BYTES : 0) + (b_tma ? Cfg::B_BYTES : 0);
          const CUtensorMap* ma = &p.tmap[pr.a.view[0]];
          const CUtensorMap* mb = &p.tmap[pr.b.view[0]];
          const bool no_load = SB200_DEBUG_BIT(p, 2);  // measurement aid
          for (int kk = wu.k0; kk < wu.k1; ++kk) {
            const bool mine = (turn == my_turn);
            if (++turn == 3u) turn = 0;
            if (!mine) {
              if (++stage == STAGES) { stage = 0; phase ^= 1u; }
              continue;
            }
            bool got = ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.wait_ns);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusProducerTimeout);
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
            uint8_t* sb = sa + Cfg::A_BYTES;
            if (ptx::elect_one()) {
              if (tx && !no_load) ptx::mbar_arrive_expect_tx(&full_bar[stage], tx);
              else ptx::mbar_arrive(&full_bar[stage]);
              if (a_tma && !no_load) ptx::tma_load_2d(sa, ma, &full_bar[stage], kk * BK, tile.i * Cfg::BM);
              if (b_tma && !no_load) {
                if (p.b_blocked) {
                  ptx::tma_load_3d(sb, mb, &full_bar[stage], 0, kk * BK, tile.j * Cfg::NBLK);
                } else {
#pragma unroll
                  for (int nb = 0; nb < Cfg::NBLK; ++nb)
                    ptx::tma_load_2d(sb + nb * Cfg::BLK_BYTES, mb, &full_bar[stage], tile.j * BN + nb * BK, kk * BK);
                }
              }
            }
            __syncwarp();
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop (see ptx::elect_one); one elected lane issues the MMAs and the commits.
    {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t free_bits = 0;
      uint32_t iter = 0;
      bool ok = true;
      for (int u = blockIdx.x; ok && u < num_units; u += gridDim.x, ++iter) {
        const WorkUnit wu = unit_of(p, u);
        const int nk = wu.k1 - wu.k0;
        const uint32_t sx = p.prog.alternate_slots ? (iter & 1u) : 0u;
        for (int ps = 0; ok && ps < nproducts; ++ps) {
          const sb200_product_t& pr = p.prog.product[ps];
          const uint32_t slot = pr.slot ^ sx;
          if (pr.wait_free) {
            bool got = ptx::mbar_wait(&slot_free[slot], ((free_bits >> slot) & 1u) ^ 1u, abort_flag, p.wait_ns);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusMmaTimeout);
              ok = false;
              break;
            }
            free_bits ^= (1u << slot);
            ptx::tc_fence_after_sync();
          }
          const uint32_t idesc = ptx::umma_idesc((ESIZE == 2 && p.bf16) ? 1u : Cfg::FMT, Cfg::BM, BN, pr.negate != 0);
          const uint32_t tmem_d = tmem_base + slot * BN;
          const bool skip_mma = SB200_DEBUG_BIT(p, 1);  // measurement aid
          // descriptors differ between stages and k-substeps only in the start-address field (low word, 16-byte units)
          const uint64_t adesc0 = ptx::umma_desc_sw128(ptx::smem_u32(smem), 16, 1024);
          const uint64_t bdesc0 =
              ptx::umma_desc_sw128(ptx::smem_u32(smem) + Cfg::A_BYTES, Cfg::BLK_BYTES, Cfg::B_SBO, Cfg::B_LAYOUT_TYPE);
          for (int kk = 0; ok && kk < nk; ++kk) {
            bool got = ptx::mbar_wait(&full_bar[stage], phase, abort_flag, p.wait_ns);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusMmaTimeout);
              ok = false;
              break;
            }
            ptx::tc_fence_after_sync();
            const uint64_t adesc_s = adesc0 + static_cast<uint64_t>((stage * Cfg::STAGE_BYTES) >> 4);
            const uint64_t bdesc_s = bdesc0 + static_cast<uint64_t>((stage * Cfg::STAGE_BYTES) >> 4);
            if (ptx::elect_one()) {
              if (!skip_mma) {
#pragma unroll
                for (int ks = 0; ks < Cfg::KSUB; ++ks) {
                  const uint64_t adesc = adesc_s + static_cast<uint64_t>((ks * 32) >> 4);
                  const uint64_t bdesc = bdesc_s + static_cast<uint64_t>((ks * Cfg::UMMA_K * 128) >> 4);
                  const uint32_t acc = (kk > 0 || ks > 0 || pr.accumulate) ? 1u : 0u;
                  if (ESIZE == 2) ptx::umma_f16(tmem_d, adesc, bdesc, idesc, acc);
                  else ptx::umma_tf32(tmem_d, adesc, bdesc, idesc, acc);
                }
              }
              ptx::umma_commit(&empty_bar[stage]);
            }
            __syncwarp();
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok && pr.commit) {
            if (ptx::elect_one()) ptx::umma_commit(&slot_full[slot]);
            __syncwarp();
          }
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;            // TMEM lane quarter this warp may read
    uint32_t full_bits = 0;
    uint32_t iter = 0;
    bool ok = true;
    for (int u = blockIdx.x; ok && u < num_units; u += gridDim.x, ++iter) {
      const WorkUnit wu = unit_of(p, u);
      const TileCoord tile = tile_of(wu.tile, p.tiles_m, p.tiles_n, p.band);
      const uint32_t sx = p.prog.alternate_slots ? (iter & 1u) : 0u;
      for (int es = 0; ok && es < p.prog.nepilogues; ++es) {
        const sb200_epilogue_t& ep = p.prog.epilogue[es];
        const SplitStep sp = split_step(ep, wu.part, wu.nparts);
        if (sp.skip) continue;
        const long long split_tile = static_cast<long long>(wu.split_idx) * 4 + sp.q;
        int* flag = p.split_flags + split_tile * 8 + quarter;
        float* split_tile_buf = p.split_buf + split_tile * (128 * BN);
        auto wait_slots = [&]() -> bool {
          for (int s = 0; s < SLOTS; ++s) {
            if ((ep.wait_full_mask >> s) & 1u) {
              const uint32_t slot = s ^ sx;
              bool got = ptx::mbar_wait(&slot_full[slot], (full_bits >> slot) & 1u, abort_flag, p.wait_ns);
              got = __all_sync(0xffffffffu, got);
              if (!got) {
                if (lane == 0) raise_abort(p, abort_flag, kStatusEpilogueTimeout);
                return false;
              }
              full_bits ^= (1u << slot);
            }
          }
          if (sp.add_partial && !wait_flag(flag, p.split_epoch, abort_flag, p.wait_ns)) {
            if (lane == 0) raise_abort(p, abort_flag, kStatusSplitTimeout);
            return false;
          }
          ptx::tc_fence_after_sync();
          return true;
        };
        const long long tile_off = static_cast<long long>(wu.ws_slot) * (128 * BN);
        const long long outer_off = static_cast<long long>(wu.tile) * (128 * BN);
        ok = epilogue_body<ESIZE, BN, Cfg::NSRC_MAX, Cfg::NSLOT_MAX, Cfg::SCALED>(p.out, p.ldo, (ep.dst & 2) ? p.out_rows2 : p.out_rows,
                                                     (ep.dst & 1) ? p.out_cols2 : p.out_cols, p.ws, ep, sx, tmem_base, quarter,
                                                     lane, tile_off, static_cast<long long>(blockIdx.x) * (128 * BN), outer_off,
                                                     tile.i * 128, tile.j * BN,
                                                     staging + (warp - 2) * kStagingWarpBytes,
                                                     sp.redirect ? split_tile_buf : nullptr,
                                                     sp.add_partial ? split_tile_buf : nullptr,
                                                     SB200_DEBUG_BIT(p, 32), wait_slots, p.alpha, p.beta, p.cin, p.ldc, nullptr,
                                                     ESIZE == 2 && p.bf16 != 0);
        if (!ok) break;
        if (sp.redirect && !p.drop_split_flags) raise_flag(flag, p.split_epoch, lane);
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          for (int s = 0; s < SLOTS; ++s)
            if ((ep.release_mask >> s) & 1u) ptx::mbar_arrive(&slot_free[s ^ sx]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ presum warps
    if (Cfg::MODE == kPresumFeed) {
      const int ptid = threadIdx.x - Cfg::FIRST_PRESUM_WARP * 32;
      constexpr int PT = Cfg::PRESUM_WARPS * 32;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; ok && u < num_units; u += gridDim.x) {
        const WorkUnit wu = unit_of(p, u);
        const TileCoord tile = tile_of(wu.tile, p.tiles_m, p.tiles_n, p.band);
        for (int ps = 0; ok && ps < nproducts; ++ps) {
          const sb200_product_t& pr = p.prog.product[ps];
          const bool a_mt = pr.a.nterms > 1;
          const bool b_mt = pr.b.nterms > 1;
          for (int kk = wu.k0; kk < wu.k1; ++kk) {
            bool got = ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.wait_ns);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusPresumTimeout);
              ok = false;
              break;
            }
            const uint32_t sa = ptx::smem_u32(smem + stage * Cfg::STAGE_BYTES);
            const uint32_t sb = sa + Cfg::A_BYTES;
            if (a_mt)
              build_operand_tile<ESIZE, Cfg::BM, 8, PT, false>(sa, 0u, pr.a, p.view, tile.i * Cfg::BM, kk * BK, ptid, p.bf16 != 0);
            if (b_mt)
              build_operand_tile<ESIZE, BK, BN * ESIZE / 16, PT, Cfg::B_SWZ32>(sb, Cfg::BLK_BYTES, pr.b, p.view, kk * BK, tile.j * BN,
                                                                  ptid, p.bf16 != 0);
            if (a_mt || b_mt) ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&full_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else if (Cfg::MODE == kPresumJob) {
      const int ptid = threadIdx.x - Cfg::FIRST_PRESUM_WARP * 32;
      constexpr int PT = Cfg::PRESUM_WARPS * 32;
      presum_job<ESIZE>(p, blockIdx.x * PT + ptid, gridDim.x * PT);
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight a bounded time to land before the shared memory is released
    uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace sb200
