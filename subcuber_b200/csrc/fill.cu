// Seeded synthetic inputs, identical on host and device.
//
// The reference driver fills A and B on the host with CUTLASS's TensorFillRandomUniform (seed 1, range
// [-4,4] for f16 and [-16,16] otherwise, 2 fractional bits; src/cuda/kernel_runner.cpp:263-275), which is
// std::rand based and cannot be reproduced on a device.  This generator is counter based instead
// (Philox4x32-10: key = seed, counter = (flat index, subsequence)), so element i of a matrix has the same
// value wherever it is produced.  Distributions:
//   0 uniform1  U[-1, 1)          24-bit mantissa draw, exact in fp32
//   1 normal    N(0, 1)           Box-Muller on two draws of the same counter (fp32 math)
//   2 harness   the reference harness' value set: multiples of 0.25 in [-R, R], R = 4 (f16) or 16
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <thread>
#include <vector>

#include "../../include/subcuber_b200.h"

namespace {

struct Philox {
  uint32_t v[4];
};

__host__ __device__ inline uint32_t mulhi32(uint32_t a, uint32_t b) {
  return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32);
}

__host__ __device__ inline Philox philox4x32_10(uint64_t index, uint32_t subseq, uint64_t seed) {
  uint32_t c0 = static_cast<uint32_t>(index), c1 = static_cast<uint32_t>(index >> 32), c2 = subseq, c3 = 0;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = mulhi32(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = mulhi32(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  Philox p;
  p.v[0] = c0; p.v[1] = c1; p.v[2] = c2; p.v[3] = c3;
  return p;
}

__host__ __device__ inline float draw(int dist, int dtype, uint64_t index, uint32_t subseq, uint64_t seed) {
  Philox p = philox4x32_10(index, subseq, seed);
  if (dist == 0) {
    float u = static_cast<float>(p.v[0] >> 8) * (1.0f / 16777216.0f);  // [0,1), exact
    return 2.0f * u - 1.0f;
  }
  if (dist == 1) {
    float u1 = (static_cast<float>(p.v[0] >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0,1]
    float u2 = static_cast<float>(p.v[1] >> 8) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
  }
  const int range = (dtype == 0 || dtype == 3) ? 4 : 16;  // 16-bit types: +-4 (sums of 16 terms stay exact in bfloat16 too)
  const uint32_t steps = static_cast<uint32_t>(8 * range + 1);
  return -static_cast<float>(range) + 0.25f * static_cast<float>(p.v[0] % steps);
}

template <typename T>
__host__ __device__ inline T convert(float x);
template <>
__host__ __device__ inline __half convert<__half>(float x) { return __float2half_rn(x); }
template <>
__host__ __device__ inline __nv_bfloat16 convert<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__host__ __device__ inline float convert<float>(float x) { return x; }
template <>
__host__ __device__ inline double convert<double>(float x) { return static_cast<double>(x); }

template <typename T>
__global__ void fill_kernel(T* out, uint64_t n, int dist, int dtype, uint32_t subseq, uint64_t seed) {
  uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) out[i] = convert<T>(draw(dist, dtype, i, subseq, seed));
}

// Every element is a pure function of its index, so the host fill splits the range over the host's threads.
template <typename T>
void fill_host_t(T* out, uint64_t n, int dist, int dtype, uint32_t subseq, uint64_t seed) {
  unsigned nt = std::thread::hardware_concurrency();
  if (nt == 0) nt = 1;
  if (nt > 64) nt = 64;
  if (n < (1u << 16)) nt = 1;
  auto range = [=](uint64_t lo, uint64_t hi) {
    for (uint64_t i = lo; i < hi; ++i) out[i] = convert<T>(draw(dist, dtype, i, subseq, seed));
  };
  if (nt == 1) {
    range(0, n);
    return;
  }
  std::vector<std::thread> pool;
  const uint64_t chunk = (n + nt - 1) / nt;
  for (unsigned t = 0; t < nt; ++t) {
    const uint64_t lo = t * chunk, hi = lo + chunk < n ? lo + chunk : n;
    if (lo < hi) pool.emplace_back(range, lo, hi);
  }
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" int sb200_fill_device(int dtype, int dist, unsigned long long seed, unsigned subsequence, void* ptr,
                                 unsigned long long count, sb200_stream_t stream) {
  if (!ptr || dist < 0 || dist > 2 || dtype < 0 || dtype > 3) return SB200_ERR_INVALID_PROBLEM;
  if (count == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int threads = 256;
  const int blocks = static_cast<int>(count / threads + 1 < 148ull * 16 ? count / threads + 1 : 148ull * 16);
  if (dtype == 0) fill_kernel<__half><<<blocks, threads, 0, s>>>(static_cast<__half*>(ptr), count, dist, dtype, subsequence, seed);
  else if (dtype == 3) fill_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>(static_cast<__nv_bfloat16*>(ptr), count, dist, dtype, subsequence, seed);
  else if (dtype == 1) fill_kernel<float><<<blocks, threads, 0, s>>>(static_cast<float*>(ptr), count, dist, dtype, subsequence, seed);
  else fill_kernel<double><<<blocks, threads, 0, s>>>(static_cast<double*>(ptr), count, dist, dtype, subsequence, seed);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb200_fill_host(int dtype, int dist, unsigned long long seed, unsigned subsequence, void* ptr,
                               unsigned long long count) {
  if (!ptr || dist < 0 || dist > 2 || dtype < 0 || dtype > 3) return SB200_ERR_INVALID_PROBLEM;
  if (dtype == 0) fill_host_t<__half>(static_cast<__half*>(ptr), count, dist, dtype, subsequence, seed);
  else if (dtype == 3) fill_host_t<__nv_bfloat16>(static_cast<__nv_bfloat16*>(ptr), count, dist, dtype, subsequence, seed);
  else if (dtype == 1) fill_host_t<float>(static_cast<float*>(ptr), count, dist, dtype, subsequence, seed);
  else fill_host_t<double>(static_cast<double*>(ptr), count, dist, dtype, subsequence, seed);
  return 0;
}
