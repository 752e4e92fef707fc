// Flags between the GPUs of one box, for the operand exchange of the multi-GPU plan (subcuber_b200/multi_gpu.py).
//
// The exchange moves operand shards between GPUs with the copy engines; what it needs from kernels is ordering only:
// "my copies into your buffer have landed" and "I am done reading my buffer, you may overwrite it".  Each of those is a
// 32-bit counter in the RECEIVER's memory that the sender raises through a peer mapping (plain stores to another GPU's
// memory over NVLink; no multicast, no TMA).  Two one-block kernels:
//   signal  raises up to kMaxPeers counters, one per peer pointer, with release semantics at system scope; stream
//           order puts it behind the copies whose completion it announces;
//   wait    waits until up to kMaxPeers local counters have reached a value.  The wait is bounded: when the limit runs
//           out it writes a status code and returns, so a peer that never arrives cannot hang this GPU.
// The reference project is single-GPU (src/cuda/kernel_runner_support.cuh:312 pins device 0) and has no counterpart.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/subcuber_b200.h"

namespace {

constexpr int kMaxPeers = SB200_MAX_PEERS;

struct PeerPointers {
  int* ptr[kMaxPeers];
};

__global__ void peer_signal_kernel(PeerPointers peers, int n, int value) {
  const int t = threadIdx.x;
  if (t < n) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peers.ptr[t]), "r"(value) : "memory");
  }
}

__global__ void peer_wait_kernel(PeerPointers flags, int n, int value, unsigned long long limit_ns, int* status) {
  const int t = threadIdx.x;
  if (t >= n) return;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  unsigned polls = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags.ptr[t]) : "memory");
    if (v >= value) return;
    if ((++polls & 15u) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 > limit_ns) {
        atomicCAS(status, 0, SB200_STATUS_PEER_TIMEOUT);
        return;
      }
    }
    __nanosleep(200);
  }
}

}  // namespace

extern "C" int sb200_peer_signal(int* const* peer_flags, int count, int value, sb200_stream_t stream) {
  if (!peer_flags || count < 0 || count > kMaxPeers) return SB200_ERR_INVALID_PROBLEM;
  if (count == 0) return 0;
  PeerPointers p;
  for (int i = 0; i < kMaxPeers; ++i) p.ptr[i] = i < count ? peer_flags[i] : nullptr;
  peer_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p, count, value);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb200_peer_wait(int* const* local_flags, int count, int value, unsigned wait_limit_us, int* status,
                               sb200_stream_t stream) {
  if (!local_flags || !status || count < 0 || count > kMaxPeers) return SB200_ERR_INVALID_PROBLEM;
  if (count == 0) return 0;
  PeerPointers p;
  for (int i = 0; i < kMaxPeers; ++i) p.ptr[i] = i < count ? local_flags[i] : nullptr;
  const unsigned long long limit_ns = wait_limit_us ? 1000ull * wait_limit_us : 2000000000ull;
  peer_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p, count, value, limit_ns, status);
  return static_cast<int>(cudaGetLastError());
}
