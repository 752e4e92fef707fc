// Host-side operator: checks, workspace layout, tensor maps, launches.  See sw_host.h.
#include "sw_host.h"

#include <cuda.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "per_device.h"
#include "sw_kernel.cuh"
#include "sw_kernel_pair.cuh"
#include "sw_programs.h"

namespace sb200 {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major view -> tensor map with a [box_rows x 128 bytes] box and 128-byte swizzle.
int make_tmap(CUtensorMap* m, int esize, const View& v, int box_rows, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return kErrInternal;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(v.cols), static_cast<cuuint64_t>(v.rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(v.ld) * esize};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / esize), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(m, dt, 2, const_cast<void*>(v.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kErrInternal;
}

// Row-major B view as a 3-D tensor [128-byte column block][row][block index] (the block stride is 128 bytes), so
// that ONE load deposits `nblk` column blocks of `box_rows` rows, each in the canonical swizzled layout, back to
// back.  Needs a column count that is a whole number of blocks: a partial last block would be read past the row end.
int make_tmap_b_blocked(CUtensorMap* m, int esize, const View& v, int box_rows, int nblk, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return kErrInternal;
  const int blk = 128 / esize;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(blk), static_cast<cuuint64_t>(v.rows),
                        static_cast<cuuint64_t>(v.cols / blk)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(v.ld) * esize, 128};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(blk), static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(nblk)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(m, dt, 3, const_cast<void*>(v.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kErrInternal;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int esize_of(DType t) { return (t == kF16 || t == kBF16) ? 2 : 4; }

struct Layout {
  int esize, bn, level;
  int mq, nq, kq;          // extents of one operand/output block of the innermost level (level 0: the whole matrix)
  int tiles_m, tiles_n, num_k;
  size_t off_status, off_pa, off_pb, off_ws[4], total;
  // level 2 only: outer presums [4][m/2][k/2], [4][k/2][n/2] and three outer chain buffers (fp32, tile-contiguous,
  // four inner quadrants each)
  size_t off_opa, off_opb, off_x[3], quadrant_floats;
  // the unit list (WorkUnit in sw_kernel.cuh)
  int workers;       // CTAs (1-CTA kernels) or CTA pairs launched
  int cap;           // most workers a launch may have (SMs, or pairs of SMs, left to this call)
  int whole_tiles;   // tiles handed out whole
  int region_tiles;  // tiles that follow, each handed out as two units (0: none)
  int region_cols;   // 1: those units are column halves of the tile (CTA pairs), 0: K-halves
  bool dynamic;      // units are drawn from a counter by whichever pair is free (else dealt round-robin)
  size_t off_split_buf, off_split_flags, split_flag_bytes;
  size_t off_panel_flags, panel_flag_bytes;  // one-launch plan: chunk counter + per-panel counters, cleared per run
};

int level_of(Variant v) { return v == kCubic ? 0 : (v == kInterleavedLevel2 ? 2 : 1); }

int sm_count() { return sm_count_of_current_device(); }

// Builds the unit list for `tiles` output tiles on at most `cap` workers (see WorkUnit in sw_kernel.cuh).
//   CTA pairs: the tiles of a last wave that is at most half full (all tiles, when there are at most half as many as
//   pairs) are cut into two column halves, independent units with a whole tile's ratio of MMA work to epilogue
//   work, so that this wave lasts half as long; with more units than pairs, units are drawn from a counter by
//   whichever pair is free (UnitCursor).
//   1-CTA kernels: tiles are dealt round-robin, and the tiles of a last wave that is at most half full are cut into
//   two K-halves.
// Measured on B200 (f16 level 1, CTA pairs) and therefore NOT done: K-halves for the last tiles of the drawn order
// (-2.5 % at 16384^3, -10 % at 8192^3) or for every tile when tiles are few (-6 % at 2048^3, -12 % at 3072^3): a K-half
// costs a whole tile's epilogue, and the halves' partial sums travel through memory.
// The fused-presum and one-launch kernels are never cut, nor are products of fewer than 8 k-steps cut along K.
void deal_tiles(Layout& L, int tiles, int cap, Variant v, bool no_split, bool pair) {
  L.workers = tiles < cap ? tiles : cap;
  L.whole_tiles = tiles;
  L.region_tiles = 0;
  L.region_cols = 0;
  L.dynamic = pair && tiles > cap;
  if (v == kFusedPresum || v == kStrassenFused || v == kMergedPresum || no_split) return;
  const int rem = tiles % cap;  // tiles of the last wave (all of them when they are fewer than the workers)
  if (rem == 0 || 2 * rem > cap) return;
  if (pair) {
    L.whole_tiles = tiles - rem;
    L.region_tiles = rem;
    L.region_cols = 1;
    const int units = L.whole_tiles + 2 * rem;
    L.workers = units < cap ? units : cap;
    L.dynamic = units > cap;
    return;
  }
  if (L.num_k < 8 || tiles <= cap) return;
  L.whole_tiles = tiles - rem;
  L.region_tiles = rem;
}

Layout make_layout(const GemmArgs& a, int cap_override = 0) {
  Layout L;
  memset(&L, 0, sizeof(L));
  L.esize = esize_of(a.dtype);
  L.bn = a.bn == 128 ? 128 : 256;
  L.level = level_of(a.variant);
  const int div = 1 << L.level;
  // Block extents: the matrices are cut at multiples of these; extents that do not divide leave the last block row /
  // column short, and the kernels treat the missing part as zeros (TMA fills loads outside a view with zeros, the
  // presum jobs and the output stores are bounded).  Column cuts keep every block row on a 16-byte boundary.
  const int vec = 16 / L.esize;
  L.mq = ceil_div(a.m, div);
  L.nq = static_cast<int>(align_up(ceil_div(a.n, div), vec));
  L.kq = static_cast<int>(align_up(ceil_div(a.k, div), vec));
  L.tiles_m = ceil_div(L.mq, a.pair ? 256 : 128);
  L.tiles_n = ceil_div(L.nq, L.bn);
  L.num_k = ceil_div(L.kq, 128 / L.esize);
  int cap = cap_override > 0 ? cap_override : sm_count();
  if (a.sm_limit > 0 && a.sm_limit < cap) cap = a.sm_limit;  // the caller keeps the other SMs for its own kernels
  if (a.pair) cap /= 2;  // one pair per two SMs
  if (cap < 1) cap = 1;
  bool no_split = a.no_split != 0;
#ifdef SB200_PROFILE
  if (getenv("SB200_NO_SPLIT")) no_split = true;  // measurement aid of profile builds
#endif
  L.cap = cap;
  deal_tiles(L, L.tiles_m * L.tiles_n, cap, a.variant, no_split, a.pair != 0);
#ifdef SB200_PROFILE
  if (const char* sc = getenv("SB200_SCHED"))  // measurement aid: 0 = round-robin deal
    if (atoi(sc) == 0) deal_tiles(L, L.tiles_m * L.tiles_n, cap, a.variant, no_split, false);
#endif
  // the status block and the flags of the cut tiles sit together at the head: one memset clears both for a run
  size_t off = 0;
  L.off_status = off;
  off += 256;
  L.off_split_flags = off;
  const int k_regions = L.region_cols ? 0 : L.region_tiles;  // tiles cut along K: flags, partial sums, extra slots
  L.split_flag_bytes = size_t(k_regions) * 4 * 8 * sizeof(int);
  off = align_up(off + L.split_flag_bytes, 256);
  L.off_panel_flags = off;
  L.panel_flag_bytes = a.variant == kMergedPresum ? align_up(size_t(1 + L.tiles_m + L.tiles_n) * sizeof(int), 256) : 0;
  off += L.panel_flag_bytes;
  if (L.level == 2) {
    L.off_opa = off;
    off = align_up(off + size_t(4) * (2 * L.mq) * (2 * L.kq) * L.esize, 256);
    L.off_opb = off;
    off = align_up(off + size_t(4) * (2 * L.kq) * (2 * L.nq) * L.esize, 256);
  }
  if (a.variant == kInterleavedPresum || a.variant == kMergedPresum || a.variant == kStrassenPresum || L.level == 2) {
    const size_t npre = a.variant == kStrassenPresum ? programs::kStrassenPresumsPerSide : 4;  // presums per side
    L.off_pa = off;
    off = align_up(off + npre * L.mq * L.kq * L.esize, 256);
    L.off_pb = off;
    off = align_up(off + npre * L.kq * L.nq * L.esize, 256);
  }
  const bool strassen = a.variant == kStrassenFused || a.variant == kStrassenPresum;
  const int nws = a.variant == kCubic ? 0 : (a.variant == kFusedPresum ? 2 : (strassen ? 3 : 4));
  const size_t tile_bytes = size_t(128) * L.bn * sizeof(float) * (a.pair ? 2 : 1);  // per tile of the grid
  const size_t quadrant_bytes = size_t(L.tiles_m) * L.tiles_n * tile_bytes;
  L.quadrant_floats = quadrant_bytes / sizeof(float);
  for (int i = 0; i < nws; ++i) {
    L.off_ws[i] = off;
    // buffer 0 (M0) is indexed by tile: the second half of every cut tile keeps its hand-off tile in an extra slot
    // behind the grid's; buffers 1..3 are indexed by worker
    // (the one-launch plan keeps M0 in a per-worker buffer too and leaves buffer 0 empty)
    const size_t bytes = i == 0 ? (a.variant == kMergedPresum ? 256 : quadrant_bytes + size_t(k_regions) * tile_bytes)
                                : size_t(L.workers) * tile_bytes;
    off = align_up(off + bytes, 256);
  }
  if (k_regions) {
    L.off_split_buf = off;
    off = align_up(off + size_t(k_regions) * 4 * tile_bytes, 256);
  }
  if (L.level == 2)
    for (int i = 0; i < 3; ++i) {
      L.off_x[i] = off;
      off = align_up(off + 4 * quadrant_bytes, 256);
    }
  L.total = off;
  return L;
}

template <typename Cfg>
int launch(const KernelParams& p, int grid, cudaStream_t stream) {
  static PerDeviceOnce attr;  // the attribute belongs to the current device's copy of the kernel
  const int arc = attr.run_once([] {
    return static_cast<int>(cudaFuncSetAttribute(sw_tile_program_kernel<Cfg>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
  });
  if (arc) return arc;
  sw_tile_program_kernel<Cfg><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// The scaled form (alpha, beta, C) has kernel instantiations of its own, for the modes whose programs write outputs
// in the plans that support it (not the fused-presum variant).
inline bool is_scaled(const KernelParams& p) { return p.alpha != 1.f || p.beta != 0.f; }

template <int ESIZE, int BN>
int launch_mode(int mode, const KernelParams& p, int grid, cudaStream_t stream) {
  constexpr int STAGES = (BN == 256) ? 4 : 6;
  if (is_scaled(p)) {
    switch (mode) {
      case kPresumNone: return launch<KernelConfig<ESIZE, BN, STAGES, kPresumNone, true>>(p, grid, stream);
      case kPresumJob: return launch<KernelConfig<ESIZE, BN, STAGES, kPresumJob, true>>(p, grid, stream);
    }
    return kErrNotSupported;
  }
  switch (mode) {
    case kPresumNone: return launch<KernelConfig<ESIZE, BN, STAGES, kPresumNone>>(p, grid, stream);
    case kPresumFeed: return launch<KernelConfig<ESIZE, BN, STAGES, kPresumFeed>>(p, grid, stream);
    case kPresumJob: return launch<KernelConfig<ESIZE, BN, STAGES, kPresumJob>>(p, grid, stream);
  }
  return kErrInternal;
}

int launch_any(int esize, int bn, int mode, const KernelParams& p, int grid, cudaStream_t stream);
int launch_any_pair(int esize, int mode, const KernelParams& p, int pairs, cudaStream_t stream);

int launch_any(int esize, int bn, int mode, const KernelParams& p, int grid, cudaStream_t stream) {
  if (bn < 0) return launch_any_pair(esize, mode, p, grid, stream);
  if (esize == 2 && bn == 256) return launch_mode<2, 256>(mode, p, grid, stream);
  if (esize == 2 && bn == 128) return launch_mode<2, 128>(mode, p, grid, stream);
  if (esize == 4 && bn == 256) return launch_mode<4, 256>(mode, p, grid, stream);
  if (esize == 4 && bn == 128) return launch_mode<4, 128>(mode, p, grid, stream);
  return kErrNotSupported;
}

template <typename Cfg>
int launch_pair(const KernelParams& p, int pairs, cudaStream_t stream) {
  static PerDeviceOnce smem_attr;  // the attribute belongs to the current device's copy of the kernel
  const int arc = smem_attr.run_once([] {
    return static_cast<int>(cudaFuncSetAttribute(sw_tile_program_pair_kernel<Cfg>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
  });
  if (arc) return arc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, sw_tile_program_pair_kernel<Cfg>, p));
}

template <int ESIZE>
int launch_pair_mode(int mode, const KernelParams& p, int pairs, cudaStream_t stream) {
  constexpr int STAGES = 6;
  if (is_scaled(p)) {
    switch (mode) {
      case kPresumNone: return launch_pair<PairConfig<ESIZE, STAGES, kPresumNone, true>>(p, pairs, stream);
      case kPresumJob: return launch_pair<PairConfig<ESIZE, STAGES, kPresumJob, true>>(p, pairs, stream);
    }
    return kErrNotSupported;
  }
  switch (mode) {
    case kPresumNone: return launch_pair<PairConfig<ESIZE, STAGES, kPresumNone>>(p, pairs, stream);
    case kPresumFeed: return launch_pair<PairConfig<ESIZE, STAGES, kPresumFeed>>(p, pairs, stream);
    case kPresumJob: return launch_pair<PairConfig<ESIZE, STAGES, kPresumJob>>(p, pairs, stream);
  }
  return kErrInternal;
}

int launch_any_pair(int esize, int mode, const KernelParams& p, int pairs, cudaStream_t stream) {
  if (esize == 2) return launch_pair_mode<2>(mode, p, pairs, stream);
  if (esize == 4) return launch_pair_mode<4>(mode, p, pairs, stream);
  return kErrNotSupported;
}

}  // namespace

namespace tc {

int can_implement(const GemmArgs& a) {
  if (a.m <= 0 || a.n <= 0 || a.k <= 0 || !a.a || !a.b || !a.d) return kErrInvalidProblem;
  if (a.dtype != kF16 && a.dtype != kF32 && a.dtype != kBF16) return kErrNotSupported;
  if (a.scaled && a.beta != 0.0 && (!a.c || (reinterpret_cast<uintptr_t>(a.c) & 15))) return kErrInvalidProblem;
  if (a.bn != 0 && a.bn != 128 && a.bn != 256) return kErrNotSupported;
  if (a.pair && a.bn == 128) return kErrNotSupported;
  if ((a.variant == kMergedPresum || a.variant == kStrassenPresum) && !a.pair) return kErrNotSupported;
  const int es = esize_of(a.dtype);
  const int vec = 16 / es;  // elements per 16 bytes
  const int div = 1 << level_of(a.variant);
  // every row must start on a 16-byte boundary (TMA base/stride rule, vector loads and stores)
  if (a.k % vec || a.n % vec) return kErrMisalignedOperand;
  // the last block row / column of every cut may be short but not empty
  const int mq = ceil_div(a.m, div);
  const int nq = static_cast<int>(align_up(ceil_div(a.n, div), vec));
  const int kq = static_cast<int>(align_up(ceil_div(a.k, div), vec));
  if (a.m - (div - 1) * mq < 1 || a.n - (div - 1) * nq < 1 || a.k - (div - 1) * kq < 1) return kErrInvalidProblem;
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) | reinterpret_cast<uintptr_t>(a.d)) & 15)
    return kErrMisalignedOperand;
  return kOk;
}

size_t workspace_bytes(const GemmArgs& a) { return make_layout(a).total; }

WorkspaceLayout workspace_layout(const GemmArgs& a) {
  WorkspaceLayout w;
  memset(&w, 0, sizeof(w));
  const Layout L = make_layout(a);
  w.status = L.off_status;
  w.presum_a = L.off_pa;
  w.presum_b = L.off_pb;
  for (int i = 0; i < 4; ++i) w.handoff[i] = L.off_ws[i];
  w.total = L.total;
  w.mq = L.mq; w.nq = L.nq; w.kq = L.kq;
  w.tiles_m = L.tiles_m; w.tiles_n = L.tiles_n; w.bn = L.bn;
  return w;
}

int deal_units(const GemmArgs& a, int sms, int* out, int max_units, int* workers) {
  const Layout L = make_layout(a, sms);
  KernelParams p;
  memset(&p, 0, sizeof(p));
  p.tiles_m = L.tiles_m; p.tiles_n = L.tiles_n; p.num_k = L.num_k;
  p.whole_tiles = L.whole_tiles; p.region_tiles = L.region_tiles; p.region_cols = L.region_cols;
  if (workers) *workers = L.workers;
  const int n = total_units(p);
  for (int u = 0; u < n && u < max_units; ++u) {
    const WorkUnit w = unit_of(p, u);
    int* o = out + size_t(u) * 10;
    o[0] = u % L.workers; o[1] = w.tile; o[2] = w.part; o[3] = w.nparts; o[4] = w.k0; o[5] = w.k1; o[6] = w.ws_slot;
    o[7] = w.split_idx; o[8] = w.col_part; o[9] = w.col_parts;
  }
  return n;
}

int launches_per_run(const GemmArgs& a) {
  if (a.variant == kInterleavedLevel2) return 14;
  return (a.variant == kInterleavedPresum || a.variant == kStrassenPresum) ? 2 : 1;  // one-launch plans: 1
}

namespace {

// One launch group over (A, B) -> D with quadrant extents (mq, nq, kq): level 0 (whole matrices, one launch), level 1
// fused (one launch) or level 1 interleaved (two launches), optionally tied into an outer recursion step.
// The 256-byte status block at the head of the workspace is cleared on the stream by every run: word 0 is the device
// status, words kUnitCounterBase + 1 .. + 14 are the unit counters of the run's launches (UnitCursor).
constexpr int kUnitCounterBase = 8;

struct LaunchSpec {
  Variant variant;
  int es, bn, pair, grid;
  int cap;                   // most workers a launch may have (a launch without products uses them all)
  int bf16;                  // 16-bit operands are bfloat16
  View a, b;                 // whole operands of this group (extents up to twice the block extents)
  int mq, nq, kq;            // extents of one block (level 0: of the whole problem)
  int tiles_m, tiles_n, num_k;
  char* out;                 // output matrix in the output type (up to 2mq x 2nq, or mq x nq at level 0), or null
  int out_rows, out_cols;    // its extents
  long long ldo;
  const char* cin;           // C input laid out like `out` (same leading dimension), or null
  float alpha, beta;
  char* presum_a;            // [4][mq][kq], interleaved only
  char* presum_b;            // [4][kq][nq]
  float* ws_inner[4];
  size_t quadrant_floats;    // floats per output quadrant in an outer chain buffer
  float* outer_dst;          // outer chain buffers ([4 quadrants][tiles][tile]) or null
  float* outer_src;
  float* outer_src2;
  float* extra_dst;
  int child;                 // group of a level-2 run (0..6), or -1: a level-1 GEMM of its own
  bool linked;
  PresumSideJob more_jobs[2];  // presum jobs of the level above, run by launch 1's presum warps
  int n_more_jobs;
  int* status;
  int whole_tiles, region_tiles, region_cols;  // the unit list (Layout)
  int dynamic;                    // CTA pairs draw their units from a counter instead of taking them round-robin
  float* split_buf;
  int* split_flags;
  int* split_epoch;          // counter shared by the launches of one run
  unsigned long long wait_ns;  // bound of every device-side wait
  int drop_split_flags;        // test aid, see GemmArgs
  int* panel_flags;            // one-launch plan: [chunk counter][tiles_m A panels][tiles_n B panels]
};

// Block (br, bc) of a matrix cut at multiples of (rows, cols): the last block row / column keeps what is left.
View block_of(const View& w, int br, int bc, int rows, int cols, int es) {
  View v;
  v.ptr = static_cast<const char*>(w.ptr) + (static_cast<long long>(br) * rows * w.ld + static_cast<long long>(bc) * cols) * es;
  v.ld = w.ld;
  v.rows = w.rows - br * rows < rows ? w.rows - br * rows : rows;
  v.cols = w.cols - bc * cols < cols ? w.cols - bc * cols : cols;
  return v;
}

#ifdef SB200_PROFILE
// Measurement aids of builds with -DSB200_PROFILE (never compiled into the product library): environment knobs for the
// raster band and the debug flags, and the in-kernel cycle counters, printed by the next launch.
void apply_tuning_aids(KernelParams& p) {
  if (const char* bd = getenv("SB200_BAND")) p.band = atoi(bd) > 0 ? atoi(bd) : p.band;
  if (const char* dbg = getenv("SB200_DEBUG_FLAGS")) p.debug_flags = atoi(dbg);
  if (const char* hm = getenv("SB200_HINT")) p.hint_mode = atoi(hm);
  if (getenv("SB200_PROF")) {
    // measurement aid: per-CTA cycle counters of the CTA-pair kernels (library built with SB200_PROFILE), printed by
    // the next call
    static long long* prof_dev = nullptr;
    static long long prof_host[4096 + 128 * 128];
    if (!prof_dev) {
      cudaMalloc(&prof_dev, sizeof(prof_host));
    } else {
      cudaDeviceSynchronize();
      cudaMemcpy(prof_host, prof_dev, sizeof(prof_host), cudaMemcpyDeviceToHost);
      double sum[8] = {0};
      int n = 0;
      for (int c = 0; c < 148; c += 2, ++n)
        for (int i = 0; i < 8; ++i) sum[i] += double(prof_host[c * 8 + i]);
      fprintf(stderr, "[prof] leader mma thread: total %.0f = wait_full %.0f + wait_free %.0f + issue %.0f + rest | "
              "producer: wait_empty %.0f issue %.0f total %.0f\n",
              sum[0] / n, sum[1] / n, sum[2] / n, sum[5] / n, sum[3] / n, sum[7] / n, sum[4] / n);
      if (prof_host[1191])
        fprintf(stderr, "[prof] tcgen05.ld 32x32 + wait: %.0f cycles per load (%lld loads)\n",
                double(prof_host[1190]) / double(prof_host[1191]), prof_host[1191]);
      fprintf(stderr, "[prof] epilogue segments (cycles, whole launch, warp 2 of CTA 0): sources %lld, tmem+add %lld, "
              "convert/stage or fp32 store %lld, output store %lld\n", prof_host[1192], prof_host[1193], prof_host[1194],
              prof_host[1195]);
      for (int es = 0; es < 16; ++es)
        if (prof_host[1200 + es * 2 + 1])
          fprintf(stderr, "[prof] epilogue step %d: %.0f cycles per call (%lld calls)\n", es,
                  double(prof_host[1200 + es * 2]) / double(prof_host[1200 + es * 2 + 1]), prof_host[1200 + es * 2 + 1]);
      {
        // start-time spread of the pairs, wave by wave
        const long long* ts = prof_host + 4096;
        for (int it = 0; it < 128; it += 4) {
          long long lo = 0, hi = 0;
          int cnt = 0;
          for (int pr = 0; pr < 74; ++pr) {
            const long long v = ts[pr * 128 + it];
            if (!v) continue;
            if (!cnt || v < lo) lo = v;
            if (!cnt || v > hi) hi = v;
            ++cnt;
          }
          if (cnt > 1) fprintf(stderr, "[skew] tile %3d of each pair: %d pairs, start spread %.1f us (first at +%.1f us)\n", it, cnt,
                               (hi - lo) * 1e-3, (lo - ts[0]) * 1e-3);
        }
        if (getenv("SB200_PROF_DUMP")) {
          // per pair: SM id of its leader CTA, then the durations of its first tiles in us
          for (int pr = 0; pr < 74; ++pr) {
            fprintf(stderr, "[dump] pair %2d sm %3lld start0 %+6.1f:", pr, prof_host[3000 + pr], (ts[pr * 128] - ts[0]) * 1e-3);
            int it = 0;
            for (; it + 1 < 24 && ts[pr * 128 + it + 1]; ++it)
              fprintf(stderr, " %6.1f", (ts[pr * 128 + it + 1] - ts[pr * 128 + it]) * 1e-3);
            fprintf(stderr, " | last unit to MMAs issued %6.1f, to last epilogue %6.1f, flag waits (CTA 0 of the pair) %6.1f\n",
                    (ts[pr * 128 + 127] - ts[pr * 128 + it]) * 1e-3, (ts[pr * 128 + 126] - ts[pr * 128 + it]) * 1e-3,
                    prof_host[2 * pr * 8 + 6] * 1e-3);
          }
        }
      }
      if (getenv("SB200_PROF_TRACE")) {
        // per k-step of one tile of CTA 0 (cycles relative to the first entry): producer saw the stage empty / issued
        // its loads, an observer saw the stage full, the MMA thread started waiting / got the stage / had issued
        const long long* t = prof_host + 2048;
        long long base = t[0];
        fprintf(stderr, "[trace] kk: prod_empty prod_issued full_seen | mma_wait_start mma_got mma_issued | load_latency\n");
        for (int kk = 0; kk < 64; ++kk, t += 8)
          fprintf(stderr, "[trace] %2d: %7lld %7lld %7lld | %7lld %7lld %7lld | %6lld\n", kk, t[0] - base, t[1] - base,
                  t[2] - base, t[3] - base, t[4] - base, t[5] - base, t[2] - t[1]);
      }
    }
    cudaMemset(prof_dev, 0, sizeof(prof_host));
    p.prof = prof_dev;
  }
}
#endif

template <typename MarkFn>
int launch_group(const LaunchSpec& s, cudaStream_t stream, MarkFn mark) {
  KernelParams p;
  memset(&p, 0, sizeof(p));
  p.status = s.status;
  p.bf16 = s.bf16;
  const int es = s.es;
  const char* A = static_cast<const char*>(s.a.ptr);
  const char* B = static_cast<const char*>(s.b.ptr);
  int rc;
  if (s.variant == kCubic) {
    for (int v = 0; v < 8; ++v) p.view[v] = s.a;
    for (int v = 8; v < 16; ++v) p.view[v] = s.b;
    p.out[0] = s.out;
    p.cin[0] = s.cin;
  } else {
    for (int q = 0; q < 4; ++q) {
      p.view[SB200_VIEW_A0 + q] = block_of(s.a, q >> 1, q & 1, s.mq, s.kq, es);
      p.view[SB200_VIEW_B0 + q] = block_of(s.b, q >> 1, q & 1, s.kq, s.nq, es);
      p.out[q] = s.out ? s.out + ((q >> 1) * s.mq * s.ldo + (q & 1) * s.nq) * es : nullptr;
      p.cin[q] = (s.out && s.cin) ? s.cin + ((q >> 1) * s.mq * s.ldo + (q & 1) * s.nq) * es : nullptr;
      if (s.variant == kInterleavedPresum || s.variant == kMergedPresum) {
        p.view[SB200_VIEW_PA0 + q] =
            View{s.presum_a + size_t(q) * s.mq * s.kq * es, static_cast<long long>(s.kq), s.mq, s.kq};
        p.view[SB200_VIEW_PB0 + q] =
            View{s.presum_b + size_t(q) * s.kq * s.nq * es, static_cast<long long>(s.nq), s.kq, s.nq};
      } else {
        p.view[SB200_VIEW_PA0 + q] = p.view[SB200_VIEW_A0 + q];
        p.view[SB200_VIEW_PB0 + q] = p.view[SB200_VIEW_B0 + q];
      }
    }
  }
  if (s.variant == kStrassenPresum) {
    // the ten presums of Strassen's original algorithm, read through the view slots the generated table names
    for (int r = 0; r < programs::kStrassenPresumsPerSide; ++r) {
      p.view[programs::strassen_presums(0)[r].view] =
          View{s.presum_a + size_t(r) * s.mq * s.kq * es, static_cast<long long>(s.kq), s.mq, s.kq};
      p.view[programs::strassen_presums(1)[r].view] =
          View{s.presum_b + size_t(r) * s.kq * s.nq * es, static_cast<long long>(s.nq), s.kq, s.nq};
    }
  }
  for (int v = 0; v < 8; ++v)
    if ((rc = make_tmap(&p.tmap[v], es, p.view[v], 128, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  // B tiles of 32-bit elements are deposited with 32-byte swizzle atoms (see KernelConfig::B_SWZ32)
  const CUtensorMapSwizzle b_swz = es == 4 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  // column blocks of B one CTA loads per k-step: BN (1-CTA kernels) or BN / 2 (CTA pairs) columns of 128 bytes each
  const int b_nblk = (s.pair ? 128 : s.bn) * es / 128;
  p.b_blocked = 1;  // needs whole 128-byte column blocks in every view
  for (int v = 8; v < 16; ++v)
    if (p.view[v].cols % (128 / es)) p.b_blocked = 0;
  for (int v = 8; v < 16; ++v) {
    rc = p.b_blocked ? make_tmap_b_blocked(&p.tmap[v], es, p.view[v], 128 / es, b_nblk, b_swz)
                     : make_tmap(&p.tmap[v], es, p.view[v], 128 / es, b_swz);
    if (rc) return rc;
    if (p.b_blocked && s.pair && s.region_cols) {
      // a column half loads half as many column blocks of a B tile
      if ((rc = make_tmap_b_blocked(&p.tmap_half_b[v - 8], es, p.view[v], 128 / es, b_nblk / 2, b_swz))) return rc;
    }
  }
  p.ldo = s.ldo;
  p.ldc = s.ldo;
  p.alpha = s.alpha;
  p.beta = s.beta;
  p.out_rows = s.out_rows < s.mq ? s.out_rows : s.mq;
  p.out_cols = s.out_cols < s.nq ? s.out_cols : s.nq;
  p.out_rows2 = s.out_rows - s.mq;
  p.out_cols2 = s.out_cols - s.nq;
  for (int i = 0; i < 4; ++i) p.ws[SB200_WS_INNER + i] = s.ws_inner[i];
  for (int q = 0; q < 4; ++q) {
    const size_t o = size_t(q) * s.quadrant_floats;
    p.ws[SB200_WS_OUTER_DST + q] = s.outer_dst ? s.outer_dst + o : nullptr;
    p.ws[SB200_WS_OUTER_SRC + q] = s.outer_src ? s.outer_src + o : nullptr;
    p.ws[SB200_WS_OUTER_SRC2 + q] = s.outer_src2 ? s.outer_src2 + o : nullptr;
    p.ws[SB200_WS_EXTRA_DST + q] = s.extra_dst ? s.extra_dst + o : nullptr;
  }
  p.tiles_m = s.tiles_m;
  p.tiles_n = s.tiles_n;
  p.num_k = s.num_k;
  p.whole_tiles = s.whole_tiles;
  p.region_tiles = s.region_tiles;
  p.region_cols = s.region_cols;
  p.split_buf = s.split_buf;
  p.split_flags = s.split_flags;
  // Raster band height in tile rows.  Units are handed out band by band, column by column inside a band, so the
  // tiles in flight cover `band` A row panels and about workers / band B column panels, and tiles that share a panel
  // start close together.  Measured on B200 at 16384^3 (f16, CTA pairs, units drawn in order): 8 rows read the least
  // from DRAM (level 0: 9.1 GB against 10.4 with 16 and 11.2 with 4; cuBLAS reads 8.9) and run fastest.
  p.band = 8;
  p.wait_ns = s.wait_ns;
  p.drop_split_flags = s.drop_split_flags;
#ifdef SB200_PROFILE
  apply_tuning_aids(p);
#endif
  if (s.variant == kInterleavedPresum || s.variant == kMergedPresum) {
    p.njobs = 2;
    for (int q = 0; q < 4; ++q) {
      p.job[0].src[q] = p.view[SB200_VIEW_A0 + q].ptr;
      p.job[1].src[q] = p.view[SB200_VIEW_B0 + q].ptr;
    }
    p.job[0].ld = s.a.ld; p.job[0].dst = s.presum_a; p.job[0].rows = s.mq; p.job[0].cols = s.kq; p.job[0].side = 0;
    p.job[0].rows2 = s.a.rows - s.mq; p.job[0].cols2 = s.a.cols - s.kq;
    p.job[1].ld = s.b.ld; p.job[1].dst = s.presum_b; p.job[1].rows = s.kq; p.job[1].cols = s.nq; p.job[1].side = 1;
    p.job[1].rows2 = s.b.rows - s.kq; p.job[1].cols2 = s.b.cols - s.nq;
    for (int j = 0; j < s.n_more_jobs; ++j) p.job[p.njobs++] = s.more_jobs[j];
  }
  if (s.variant == kStrassenPresum) {
    // two table-driven presum jobs over the raw quadrants (view slots 1 and 9 hold presums in this plan)
    p.njobs = 2;
    for (int side = 0; side < 2; ++side) {
      PresumSideJob& j = p.job[side];
      const View& whole = side == 0 ? s.a : s.b;
      const int rows = side == 0 ? s.mq : s.kq, cols = side == 0 ? s.kq : s.nq;
      for (int q = 0; q < 4; ++q) j.src[q] = block_of(whole, q >> 1, q & 1, rows, cols, es).ptr;
      j.ld = whole.ld; j.dst = side == 0 ? s.presum_a : s.presum_b; j.rows = rows; j.cols = cols; j.side = side;
      j.rows2 = whole.rows - rows; j.cols2 = whole.cols - cols;
      j.npairs = programs::kStrassenPresumsPerSide;
      for (int r = 0; r < j.npairs; ++r) {
        const programs::PresumPair& pp = programs::strassen_presums(side)[r];
        j.pair_q[r][0] = static_cast<signed char>(pp.q0); j.pair_c[r][0] = static_cast<signed char>(pp.c0);
        j.pair_q[r][1] = static_cast<signed char>(pp.q1); j.pair_c[r][1] = static_cast<signed char>(pp.c1);
      }
    }
  }
  const int bn_sel = s.pair ? -1 : s.bn;  // -1 routes launch_any to the CTA-pair kernels (grid = pairs)
  switch (s.variant) {
    case kCubic:
      p.prog = programs::level0();
      p.split_epoch = ++*s.split_epoch;
      p.unit_counter = s.dynamic ? s.status + kUnitCounterBase + p.split_epoch : nullptr;
      rc = launch_any(es, bn_sel, kPresumNone, p, s.grid, stream);
      break;
    case kFusedPresum:
      p.prog = programs::level1_fused();
      rc = launch_any(es, bn_sel, kPresumFeed, p, s.grid, stream);
      break;
    case kStrassenFused:
      p.prog = programs::level1_strassen();
      rc = launch_any(es, bn_sel, kPresumFeed, p, s.grid, stream);
      break;
    case kStrassenPresum: {
      // launch 1: no products, the presum warps of every worker materialise the ten presums; launch 2: the products
      const sb200_program_t products = programs::level1_strassen_presum();
      const int whole = p.whole_tiles, region = p.region_tiles;
      memset(&p.prog, 0, sizeof(p.prog));
      p.whole_tiles = 0;
      p.region_tiles = 0;
      p.unit_counter = nullptr;
      p.split_epoch = ++*s.split_epoch;
      rc = launch_any(es, bn_sel, kPresumJob, p, s.cap, stream);
      if (rc) return rc;
      if ((rc = mark())) return rc;
      p.prog = products;
      p.whole_tiles = whole;
      p.region_tiles = region;
      p.njobs = 0;
      p.split_epoch = ++*s.split_epoch;
      p.unit_counter = s.dynamic ? s.status + kUnitCounterBase + p.split_epoch : nullptr;
      // this program's epilogue steps sum two TMEM slots: of the kernels that read operands by TMA only, the
      // configuration with presum warps is the one compiled for that (its presum warps find no job here)
      rc = launch_any(es, bn_sel, kPresumJob, p, s.grid, stream);
      break;
    }
    case kMergedPresum:
      // one launch: the presum warps publish the presums panel by panel in the order of the tile raster
      p.prog = programs::level1_merged();
      p.split_epoch = ++*s.split_epoch;
      p.unit_counter = s.dynamic ? s.status + kUnitCounterBase + p.split_epoch : nullptr;
      p.panels.enabled = 1;
      p.panels.chunk_k = 512;
      p.panels.chunks = ceil_div(s.kq, p.panels.chunk_k);
      p.panels.panel_rows = s.pair ? 256 : 128;
      p.panels.panel_cols = s.bn;
      p.panels.group_cols = s.pair ? ceil_div(s.grid, p.band) : 0;  // s.grid = pairs for the CTA-pair kernels
#ifdef SB200_PROFILE
      if (const char* g = getenv("SB200_PANEL_GROUP")) p.panels.group_cols = atoi(g);
#endif
      p.panels.next_chunk = s.panel_flags;
      p.panels.ready_a = s.panel_flags + 1;
      p.panels.ready_b = s.panel_flags + 1 + s.tiles_m;
      rc = launch_any(es, bn_sel, kPresumJob, p, s.grid, stream);
      break;
    case kInterleavedPresum: {
      p.prog = s.linked ? programs::level2_launch(s.child, 1) : programs::level1_first();
      p.split_epoch = ++*s.split_epoch;
      p.unit_counter = s.dynamic ? s.status + kUnitCounterBase + p.split_epoch : nullptr;
      rc = launch_any(es, bn_sel, kPresumJob, p, s.grid, stream);
      if (rc) return rc;
      if ((rc = mark())) return rc;
      p.prog = s.linked ? programs::level2_launch(s.child, 2) : programs::level1_second();
      p.split_epoch = ++*s.split_epoch;
      p.unit_counter = s.dynamic ? s.status + kUnitCounterBase + p.split_epoch : nullptr;
      p.njobs = 0;
#ifdef SB200_PROFILE
      if (getenv("SB200_SECOND_AS_JOB")) {  // measurement aid: the second launch in the 384-thread configuration
        rc = launch_any(es, bn_sel, kPresumJob, p, s.grid, stream);
        break;
      }
#endif
      rc = launch_any(es, bn_sel, kPresumNone, p, s.grid, stream);
      break;
    }
    default:
      return kErrNotSupported;
  }
  if (rc) return rc;
  return mark();
}

}  // namespace

int run(const GemmArgs& a, void* workspace, size_t workspace_size, cudaStream_t stream) {
  int rc = tc::can_implement(a);
  if (rc) return rc;
  const Layout L = make_layout(a);
  if (!workspace) return kErrWorkspaceNull;
  if (workspace_size < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return kErrWorkspaceNull;
  char* wsb = static_cast<char*>(workspace);
  const int es = L.esize;

  int* status = reinterpret_cast<int*>(wsb + L.off_status);
  // status, unit counters, split flags, panel counters: adjacent, one memset
  cudaError_t ce = cudaMemsetAsync(status, 0, 256 + align_up(L.split_flag_bytes, 256) + L.panel_flag_bytes, stream);
  if (ce != cudaSuccess) return static_cast<int>(ce);

  int nev = 0;
  auto mark = [&]() -> int {
    if (!a.events) return 0;
    return static_cast<int>(cudaEventRecord(a.events[nev++], stream));
  };

  LaunchSpec s;
  memset(&s, 0, sizeof(s));
  s.es = es;
  s.bf16 = a.dtype == kBF16 ? 1 : 0;
  s.bn = L.bn;
  s.pair = a.pair;
  s.grid = L.workers;
  s.cap = L.cap;
  int epoch = 0;
  s.split_epoch = &epoch;
  s.whole_tiles = L.whole_tiles;
  s.region_tiles = L.region_tiles;
  s.region_cols = L.region_cols;
  s.dynamic = L.dynamic;
  if (L.region_tiles && !L.region_cols) {
    s.split_buf = reinterpret_cast<float*>(wsb + L.off_split_buf);
    s.split_flags = reinterpret_cast<int*>(wsb + L.off_split_flags);
  }
  s.mq = L.mq; s.nq = L.nq; s.kq = L.kq;
  s.tiles_m = L.tiles_m; s.tiles_n = L.tiles_n; s.num_k = L.num_k;
  s.presum_a = wsb + L.off_pa;
  s.presum_b = wsb + L.off_pb;
  for (int i = 0; i < 4; ++i) s.ws_inner[i] = reinterpret_cast<float*>(wsb + L.off_ws[i]);
  s.quadrant_floats = L.quadrant_floats;
  s.status = status;
  s.panel_flags = reinterpret_cast<int*>(wsb + L.off_panel_flags);
  s.wait_ns = a.wait_limit_us > 0 ? 1000ull * static_cast<unsigned long long>(a.wait_limit_us) : 2000000000ull;
  s.drop_split_flags = a.drop_split_flags;
  s.alpha = a.scaled ? static_cast<float>(a.alpha) : 1.f;
  s.beta = a.scaled ? static_cast<float>(a.beta) : 0.f;
  const char* Cin = (a.scaled && a.beta != 0.0) ? static_cast<const char*>(a.c) : nullptr;

  if ((rc = mark())) return rc;
  if (L.level < 2) {
    s.variant = a.variant;
    s.a = View{a.a, static_cast<long long>(a.k), a.m, a.k};
    s.b = View{a.b, static_cast<long long>(a.n), a.k, a.n};
    s.out = static_cast<char*>(a.d);
    s.out_rows = a.m;
    s.out_cols = a.n;
    s.cin = Cin;
    s.ldo = a.n;
    return launch_group(s, stream, mark);
  }

  // ---- level 2: seven level-1 groups over half-size operands (the reference's StrassenGemmLevel2 wires seven
  // child operators the same way, include/cutlass/gemm/device/strassen_gemm.h:1300-2008), chained through three
  // fp32 buffers instead of interim matrices in the output type.
  const int mh = 2 * L.mq, nh = 2 * L.nq, kh = 2 * L.kq;
  const char* A = static_cast<const char*>(a.a);
  const char* B = static_cast<const char*>(a.b);
  char* D = static_cast<char*>(a.d);
  const long long lda = a.k, ldb = a.n, ldd = a.n;
  char* opa = wsb + L.off_opa;
  char* opb = wsb + L.off_opb;
  float* X[3];
  for (int i = 0; i < 3; ++i) X[i] = reinterpret_cast<float*>(wsb + L.off_x[i]);
  const View whole_a{A, lda, a.m, a.k}, whole_b{B, ldb, a.k, a.n};
  auto operand_a = [&](int code) -> View {
    if (code < 4) return block_of(whole_a, code >> 1, code & 1, mh, kh, es);
    return View{opa + size_t(code - 4) * mh * kh * es, static_cast<long long>(kh), mh, kh};
  };
  auto operand_b = [&](int code) -> View {
    if (code < 4) return block_of(whole_b, code >> 1, code & 1, kh, nh, es);
    return View{opb + size_t(code - 4) * kh * nh * es, static_cast<long long>(nh), kh, nh};
  };
  const programs::Level2Child* children = programs::level2_children();
  s.variant = kInterleavedPresum;
  s.linked = true;
  for (int c = 0; c < 7; ++c) {
    const programs::Level2Child& ch = children[c];
    s.a = operand_a(ch.a);
    s.b = operand_b(ch.b);
    s.child = c;
    const long long out_off = ch.out_quadrant >= 0 ? ((ch.out_quadrant >> 1) * mh * ldd + (ch.out_quadrant & 1) * nh) * es : 0;
    s.out = ch.out_quadrant >= 0 ? D + out_off : nullptr;
    s.out_rows = (ch.out_quadrant >= 0 && (ch.out_quadrant >> 1)) ? a.m - mh : mh;
    s.out_cols = (ch.out_quadrant >= 0 && (ch.out_quadrant & 1)) ? a.n - nh : nh;
    s.cin = (ch.out_quadrant >= 0 && Cin) ? Cin + out_off : nullptr;
    s.ldo = ldd;
    s.outer_dst = ch.dst >= 0 ? X[ch.dst] : nullptr;
    s.outer_src = ch.src >= 0 ? X[ch.src] : nullptr;
    s.outer_src2 = ch.src2 >= 0 ? X[ch.src2] : nullptr;
    s.extra_dst = ch.extra_dst >= 0 ? X[ch.extra_dst] : nullptr;
    // The outer presums are formed by the presum warps of the first two groups, which read only raw quadrants: the A
    // side rides on m0's first launch, the B side on m1's; the first group that reads them (m2) starts afterwards.
    s.n_more_jobs = 0;
    if (c < 2) {
      PresumSideJob& j = s.more_jobs[0];
      for (int q = 0; q < 4; ++q)
        j.src[q] = c == 0 ? static_cast<const void*>(A + ((q >> 1) * mh * lda + (q & 1) * kh) * es)
                          : static_cast<const void*>(B + ((q >> 1) * kh * ldb + (q & 1) * nh) * es);
      j.ld = c == 0 ? lda : ldb;
      j.dst = c == 0 ? opa : opb;
      j.rows = c == 0 ? mh : kh;
      j.cols = c == 0 ? kh : nh;
      j.rows2 = c == 0 ? a.m - mh : a.k - kh;
      j.cols2 = c == 0 ? a.k - kh : a.n - nh;
      j.side = c;
      s.n_more_jobs = 1;
    }
    if ((rc = launch_group(s, stream, mark))) return rc;
  }
  return kOk;
}

}  // namespace tc

int read_status(void* workspace, cudaStream_t stream) {
  int st = 0;
  cudaError_t e = cudaMemcpyAsync(&st, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  return st;
}

}  // namespace sb200
