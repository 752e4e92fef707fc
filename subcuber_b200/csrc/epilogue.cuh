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
#include "ptx.cuh"
#include "tile_program.h"

namespace sb200 {

constexpr int kStagingRowBytes = 144;
constexpr int kStagingWarpBytes = 32 * kStagingRowBytes;
constexpr int kStagingBytes = 4 * kStagingWarpBytes;

struct KernelParams;

// `wait_slots()` blocks until the slots in ep.wait_full_mask are ready and returns false when the wait was given up.
template <int ESIZE, int BN, int NSRC_MAX, typename WaitFn>
__device__ __forceinline__ bool epilogue_body(void* const* out, long long ldo, int out_rows, int out_cols,
                                              float* const* ws, const sb200_epilogue_t& ep, uint32_t sx,
                                              uint32_t tmem_base, int quarter, int lane, long long tile_off,
                                              int grow_tile, int gcol_tile, uint32_t staging_warp, bool skip_body,
                                              WaitFn wait_slots) {
  if (skip_body) return wait_slots();  // measurement aid
  constexpr int NCHUNK = BN / 32;
  const int row = quarter * 32 + lane;
  const int nsrc = ep.nsrc;
  const float4* srcp[NSRC_MAX];
#pragma unroll
  for (int t = 0; t < NSRC_MAX; ++t)
    srcp[t] = (t < nsrc) ? reinterpret_cast<const float4*>(ws[ep.src[t]] + tile_off) + row : nullptr;
  float4 nxt[NSRC_MAX][8];
#pragma unroll
  for (int t = 0; t < NSRC_MAX; ++t)
    if (t < nsrc) {
#pragma unroll
      for (int q = 0; q < 8; ++q) nxt[t][q] = srcp[t][q * 128];
    }
  float4* dstp = (ep.dst_kind == 1) ? reinterpret_cast<float4*>(ws[ep.dst] + tile_off) + row : nullptr;
  char* outp = (ep.dst_kind == 1) ? nullptr : static_cast<char*>(out[ep.dst]);
  if (!wait_slots()) return false;

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
#pragma unroll
    for (int t = 0; t < SB200_MAX_SLOT_TERMS; ++t) {
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
    if (ep.dst_kind == 1) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        dstp[(c * 8 + q) * 128] = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    } else if (ESIZE == 2) {
      // 32 columns = 64 bytes per row per chunk; two chunks fill a 128-byte staging row
      const uint32_t wr = staging_warp + lane * kStagingRowBytes + (c & 1) * 64;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int q = 0; q < 4; ++q) h[q] = __floats2half2_rn(acc[g * 8 + 2 * q], acc[g * 8 + 2 * q + 1]);
        ptx::sts_v4(wr + g * 16, o);
      }
      if (c & 1) {
        __syncwarp();
        const int col = gcol_tile + (c - 1) * 32 + (lane & 7) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r_in = i * 4 + (lane >> 3);
          const int grow = grow_tile + quarter * 32 + r_in;
          const uint4 v = ptx::lds_v4(staging_warp + r_in * kStagingRowBytes + (lane & 7) * 16);
          if (grow < out_rows && col < out_cols)
            *reinterpret_cast<uint4*>(outp + (static_cast<long long>(grow) * ldo + col) * 2) = v;
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
          *reinterpret_cast<uint4*>(outp + (static_cast<long long>(grow) * ldo + col) * 4) = v;
      }
      __syncwarp();
    }
  }
  return true;
}

}  // namespace sb200
