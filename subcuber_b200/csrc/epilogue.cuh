// Postsum epilogue body shared by the 1-CTA and the CTA-pair tile-program kernels.
//
// One call handles one epilogue step of a tile program for one warp: the warp owns 32 rows (one TMEM lane
// quarter) of the CTA's 128-row accumulator and walks the BN columns in chunks of 32.  Per chunk it
//   1. sums the fp32 hand-off tiles the step lists (loaded one chunk AHEAD, so their latency overlaps the work on
//      the current chunk; the first chunk is requested BEFORE the warp waits for the step's TMEM slots, so it
//      overlaps the product that is still running),
//   2. adds / subtracts the TMEM slots (tcgen05.ld 32 lanes x 32 columns),
//   3. writes either an fp32 hand-off tile or the output in the output type.
//
// Layouts chosen for coalescing:
//   * hand-off tiles are private to the CTA that writes them, so they use the order
//     [chunk c][float4 q of the chunk][row][4 floats]: a warp-wide load or store of float4 q touches 512
//     contiguous bytes.
//   * the output is row-major in global memory while a thread owns a row, so rows go through a per-warp staging
//     area in shared memory (32 rows x 128 payload bytes, 144-byte pitch = conflict-free 16-byte accesses) and leave
//     as full 128-byte row segments: each warp-wide store writes 4 rows x 128 contiguous bytes.
#pragma once
#include <cuda_bf16.h>

#include "ptx.cuh"
#include "tile_program.h"

namespace sb200 {

constexpr int kStagingRowBytes = 144;
constexpr int kStagingWarpBytes = 32 * kStagingRowBytes;
constexpr int kStagingBytes = 4 * kStagingWarpBytes;

struct KernelParams;

// ---------------------------------------------------------------------------------------------------------------
// K-split tiles (WorkUnit in sw_kernel.cuh): what an epilogue step does in each half.
//   * a step that leaves the tile (output quadrant, or a buffer of the level above: index >= SB200_WS_OUTER_DST)
//     - first half: sums its slots and level-1 hand-offs only and writes the partial sum to the split buffer
//       (`redirect`), then raises the flag of its warp;
//     - second half: waits for that flag and adds the partial sum (`add_partial`) to everything the step lists;
//   * an extra step of the level above (no slots, reads ws[4 + q]) runs in the second half only (`skip`);
//   * steps between level-1 hand-off tiles run in both halves on private tiles.
struct SplitStep {
  bool skip, redirect, add_partial;
  int q;  // output quadrant the step belongs to
};
__device__ __forceinline__ SplitStep split_step(const sb200_epilogue_t& ep, int part, int nparts) {
  SplitStep s;
  s.skip = s.redirect = s.add_partial = false;
  s.q = 0;
  if (nparts == 1) return s;
  const bool leaves = ep.dst_kind == 0 || ep.dst >= SB200_WS_OUTER_DST;
  const bool extra = ep.nslots == 0 && ep.nsrc > 0 && ep.src[0] >= SB200_WS_OUTER_DST;
  s.q = (ep.dst_kind == 0 ? ep.dst : ep.dst - SB200_WS_OUTER_DST) & 3;
  if (part == 0) {
    s.skip = extra;
    s.redirect = leaves && !extra;
  } else {
    s.add_partial = leaves && !extra;
  }
  return s;
}

// Every lane has written its part of the partial tile: make the writes visible device-wide, then publish.
__device__ __forceinline__ void raise_flag(int* flag, int epoch, int lane) {
  __threadfence();
  __syncwarp();
  if (lane == 0) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
}
// Bounded wait (`limit_ns`, or until another thread of the CTA gives up) for the flag of the matching warp of the other
// half.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, volatile int* abort_flag, uint64_t limit_ns) {
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t polls = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    const bool all_ready = __all_sync(0xffffffffu, v == epoch);
    if (all_ready) return true;
    if ((++polls & 63u) == 0) {
      const bool give_up = *abort_flag != 0 || ptx::globaltimer_ns() - t0 > limit_ns;
      if (__any_sync(0xffffffffu, give_up)) return false;
    }
    __nanosleep(100);
  }
}

// `wait_slots()` blocks until the slots in ep.wait_full_mask are ready (and, for the second half of a split tile,
// until the first half's partial sum is published) and returns false when the wait was given up.
//   tile_off / cta_off / outer_off: float offsets into the hand-off buffers.  Buffer 0 (M0) crosses from launch 1 to
//                         launch 2 and is indexed by the unit's tile slot; buffers 1..3 live only within one tile
//                         program, so they are indexed by the CTA: the same 128 x BN tile is rewritten for every
//                         tile the CTA computes and stays in L2 instead of streaming through HBM; buffers of the
//                         level above (index >= 4) are indexed by the tile
//   NSRC_MAX / NSLOT_MAX: most fp32 sources / TMEM slots a step of the programs this kernel runs can list
//   SCALED: outputs are alpha * sum + beta * C (separate kernel instantiations, so that the plain D = A * B kernels
//           do not carry the registers of this path)
//   redirect: non-null = first half of a split tile: write the fp32 partial sum there, skip the outer sources
//   late_src: non-null = second half: one more fp32 source, readable only after wait_slots()
template <int ESIZE, int BN, int NSRC_MAX, int NSLOT_MAX, bool SCALED, typename WaitFn>
__device__ __forceinline__ bool epilogue_body(void* const* out, long long ldo, int out_rows, int out_cols,
                                              float* const* ws, const sb200_epilogue_t& ep, uint32_t sx,
                                              uint32_t tmem_base, int quarter, int lane, long long tile_off,
                                              long long cta_off, long long outer_off, int grow_tile, int gcol_tile, uint32_t staging_warp,
                                              float* redirect, const float* late_src, bool skip_body,
                                              WaitFn wait_slots, float alpha = 1.f, float beta = 0.f,
                                              const void* const* cin = nullptr, long long ldc = 0,
                                              long long* prof = nullptr, bool bf16 = false, int nchunk = BN / 32) {
#ifdef SB200_PROFILE
  if (skip_body) return wait_slots();  // measurement aid
#endif
  const int NCHUNK = nchunk;  // 32-column chunks of the unit: BN / 32, or half of that for a column half of a tile
  const int row = quarter * 32 + lane;
  // sources: the step's list (outer sources, which come last, are left to the second half of a split tile), then the
  // late source
  int nsrc = ep.nsrc;
  if (redirect)
    while (nsrc > 0 && ep.src[nsrc - 1] >= SB200_WS_OUTER_DST) --nsrc;
  const int nearly = nsrc;  // sources that may be requested before the wait
  if (late_src) ++nsrc;
  const float4* srcp[NSRC_MAX];
#pragma unroll
  for (int t = 0; t < NSRC_MAX; ++t) {
    srcp[t] = nullptr;
    if (t < nearly) {
      const int id = ep.src[t];
      srcp[t] = reinterpret_cast<const float4*>(ws[id] + (id == 0 ? tile_off : (id < SB200_WS_OUTER_DST ? cta_off : outer_off))) + row;
    } else if (t == nearly && late_src) {
      srcp[t] = reinterpret_cast<const float4*>(late_src) + row;
    }
  }
  float4 nxt[NSRC_MAX][8];
#pragma unroll
  for (int t = 0; t < NSRC_MAX; ++t)
    if (t < nearly) {
#pragma unroll
      for (int q = 0; q < 8; ++q) nxt[t][q] = srcp[t][q * 128];
    }
  const bool to_fp32 = redirect != nullptr || ep.dst_kind == 1;
  float4* dstp = nullptr;
  if (redirect) dstp = reinterpret_cast<float4*>(redirect) + row;
  else if (ep.dst_kind == 1)
    dstp = reinterpret_cast<float4*>(ws[ep.dst] +
                                     (ep.dst == 0 ? tile_off : (ep.dst < SB200_WS_OUTER_DST ? cta_off : outer_off))) + row;
  char* outp = to_fp32 ? nullptr : static_cast<char*>(out[ep.dst]);
  if (!wait_slots()) return false;
#pragma unroll
  for (int t = 0; t < NSRC_MAX; ++t)
    if (t >= nearly && t < nsrc) {
#pragma unroll
      for (int q = 0; q < 8; ++q) nxt[t][q] = srcp[t][q * 128];
    }

  uint32_t rn[32];
  const uint32_t tmem_slot0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (ep.slot[0] ^ sx) * BN;
  if (ep.nslots > 0) ptx::tmem_ld_32x32(tmem_slot0, rn);
#ifdef SB200_PROFILE_EPILOGUE
#define SB200_SEG(i) { const long long tn = clock64(); seg[i] += tn - tseg; tseg = tn; }
  long long seg[5] = {0, 0, 0, 0, 0};
  long long tseg = clock64();
#else
#define SB200_SEG(i)
#endif
#pragma unroll 1
  for (int c = 0; c < NCHUNK; ++c) {
    float acc[32];
#pragma unroll
    for (int q = 0; q < 32; ++q) acc[q] = 0.f;
#pragma unroll
    for (int t = 0; t < NSRC_MAX; ++t)
      if (t < nsrc) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          acc[4 * q + 0] += nxt[t][q].x;
          acc[4 * q + 1] += nxt[t][q].y;
          acc[4 * q + 2] += nxt[t][q].z;
          acc[4 * q + 3] += nxt[t][q].w;
        }
      }
    if (c + 1 < NCHUNK) {
#pragma unroll
      for (int t = 0; t < NSRC_MAX; ++t)
        if (t < nsrc) {
#pragma unroll
          for (int q = 0; q < 8; ++q) nxt[t][q] = srcp[t][((c + 1) * 8 + q) * 128];
        }
    }
    SB200_SEG(0)
    // slot 0 of the step: its chunk was requested one iteration ago (or before the loop); take it, then request the
    // next chunk at once so that the TMEM read overlaps the conversion and the stores below
    if (ep.nslots > 0) {
#ifdef SB200_PROFILE_EPILOGUE
      const long long tl0 = clock64();
#endif
      ptx::tmem_ld_wait();
#ifdef SB200_PROFILE_EPILOGUE
      seg[4] += clock64() - tl0;
#endif
      if (ep.slot_sign[0] > 0) {
#pragma unroll
        for (int q = 0; q < 32; ++q) acc[q] += __uint_as_float(rn[q]);
      } else {
#pragma unroll
        for (int q = 0; q < 32; ++q) acc[q] -= __uint_as_float(rn[q]);
      }
      if (c + 1 < NCHUNK) ptx::tmem_ld_32x32(tmem_slot0 + (c + 1) * 32, rn);
    }
#pragma unroll
    for (int t = 1; t < NSLOT_MAX; ++t) {
      if (t < ep.nslots) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (ep.slot[t] ^ sx) * BN + c * 32, r);
        ptx::tmem_ld_wait();
        if (ep.slot_sign[t] > 0) {
#pragma unroll
          for (int q = 0; q < 32; ++q) acc[q] += __uint_as_float(r[q]);
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q) acc[q] -= __uint_as_float(r[q]);
        }
      }
    }
    SB200_SEG(1)
    if (SCALED && !to_fp32) {
      // general form D = alpha * sum + beta * C: this thread's row, 32 columns, read 16 bytes at a time
      const char* cp = (beta != 0.f && cin) ? static_cast<const char*>(cin[ep.dst]) : nullptr;
      const int grow = grow_tile + row;
      const int gcol = gcol_tile + c * 32;
#pragma unroll
      for (int v = 0; v < 32 * ESIZE / 16; ++v) {
        constexpr int EPV = 16 / ESIZE;
        float cv[EPV];
#pragma unroll
        for (int e = 0; e < EPV; ++e) cv[e] = 0.f;
        if (cp && grow < out_rows && gcol + v * EPV < out_cols) {
          const uint4 raw = *reinterpret_cast<const uint4*>(cp + (static_cast<long long>(grow) * ldc + gcol + v * EPV) * ESIZE);
          if (ESIZE == 2) {
            const uint32_t* h = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = bf16 ? make_float2(__uint_as_float(h[e] << 16), __uint_as_float(h[e] & 0xffff0000u))
                                    : __half22float2(*reinterpret_cast<const __half2*>(&h[e]));
              cv[(2 * e) % EPV] = f.x;
              cv[(2 * e + 1) % EPV] = f.y;
            }
          } else {
            cv[0] = __uint_as_float(raw.x);
            cv[1] = __uint_as_float(raw.y);
            cv[2 % EPV] = __uint_as_float(raw.z);
            cv[3 % EPV] = __uint_as_float(raw.w);
          }
        }
#pragma unroll
        for (int e = 0; e < EPV; ++e) acc[v * EPV + e] = alpha * acc[v * EPV + e] + beta * cv[e];
      }
    }
    if (to_fp32) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        dstp[(c * 8 + q) * 128] = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    } else if (ESIZE == 2) {
      // 32 columns = 64 bytes per row per chunk; two chunks fill a 128-byte staging row
      const uint32_t wr = staging_warp + lane * kStagingRowBytes + (c & 1) * 64;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        if (bf16) {
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(acc[g * 8 + 2 * q], acc[g * 8 + 2 * q + 1]);
        } else {
          __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
          for (int q = 0; q < 4; ++q) h[q] = __floats2half2_rn(acc[g * 8 + 2 * q], acc[g * 8 + 2 * q + 1]);
        }
        ptx::sts_v4(wr + g * 16, o);
      }
      SB200_SEG(2)
      if (c & 1) {
        __syncwarp();
        const int col = gcol_tile + (c - 1) * 32 + (lane & 7) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r_in = i * 4 + (lane >> 3);
          const int grow = grow_tile + quarter * 32 + r_in;
          const uint4 v = ptx::lds_v4(staging_warp + r_in * kStagingRowBytes + (lane & 7) * 16);
          if (grow < out_rows && col < out_cols)
            ptx::stg_cs_v4(outp + (static_cast<long long>(grow) * ldo + col) * 2, v);
        }
        __syncwarp();
      }
    } else {
      // 32 columns = 128 bytes per row per chunk
      const uint32_t wr = staging_warp + lane * kStagingRowBytes;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        uint4 o;
        o.x = __float_as_uint(acc[4 * g]);
        o.y = __float_as_uint(acc[4 * g + 1]);
        o.z = __float_as_uint(acc[4 * g + 2]);
        o.w = __float_as_uint(acc[4 * g + 3]);
        ptx::sts_v4(wr + g * 16, o);
      }
      __syncwarp();
      const int col = gcol_tile + c * 32 + (lane & 7) * 4;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r_in = i * 4 + (lane >> 3);
        const int grow = grow_tile + quarter * 32 + r_in;
        const uint4 v = ptx::lds_v4(staging_warp + r_in * kStagingRowBytes + (lane & 7) * 16);
        if (grow < out_rows && col < out_cols)
          ptx::stg_cs_v4(outp + (static_cast<long long>(grow) * ldo + col) * 4, v);
      }
      __syncwarp();
    }
    SB200_SEG(3)
  }
#ifdef SB200_PROFILE_EPILOGUE
  if (prof && lane == 0) {
    prof[0] += seg[4];
    prof[1] += NCHUNK * ep.nslots;
    for (int i = 0; i < 4; ++i) prof[2 + i] += seg[i];
  }
#endif
  return true;
}

}  // namespace sb200
