// A GEMM entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc around a GEMM: a serving loop that has handed all of its
// device memory to its own pool and forbids foreign allocations; code that runs while another stream of the
// process must not be stalled (cudaMalloc and cudaFree synchronise the whole device); plugin sandboxes that
// grant a library no allocation rights at all.  The level-1 kernels need scratch memory (the eight presum
// buffers and two fp32 hand-off buffers), which every other entry point takes from the caller or allocates.
// This one keeps that scratch in a fixed array inside the library image instead.
//
// Cost and limits, all deliberate:
//  * the array occupies SB200_STATIC_SCRATCH_BYTES of device memory on EVERY GPU that loads the library, from
//    the first use of this file's code on that GPU until the process exits;
//  * problems whose scratch does not fit are refused with SB200_ERR_SCRATCH_TOO_LARGE, nothing is launched;
//  * there is one array per GPU: every call reuses it, finds the previous call's bytes in it, and two calls
//    whose kernels overlap on the GPU (different streams, or one stream per thread) corrupt each other.
//    Calls must be ordered one after the other on the device.
//
// Host code cannot use the array's name as an address: in host code the name denotes a host-side shadow
// symbol, and a kernel handed that value would fault or, where the GPU can reach host memory, scribble over
// the wrong bytes.  The device address is obtained with cudaGetSymbolAddress, once per device, with that
// device current, and cached.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

#include "../../include/subcuber_b200.h"
#include "sw_host.h"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[SB200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices];  // device address of g_static_scratch per device ordinal, 0 = not looked up yet
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device (looked up on the first call per device).
int scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return SB200_ERR_NOT_SUPPORTED;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (!p || (reinterpret_cast<uintptr_t>(p) & 255)) return SB200_ERR_INTERNAL;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int sb200_gemm_f16_sw_static_scratch(const void* a, const void* b, void* d, int m, int n, int k,
                                                sb200_stream_t stream, int wait) {
  sb200::GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.dtype = sb200::kF16;
  g.variant = sb200::kInterleavedPresum;
  g.m = m;
  g.n = n;
  g.k = k;
  g.a = a;
  g.b = b;
  g.d = d;
  g.bn = 256;
  g.no_split = 1;  // no tile is cut along K: the scratch stays small and its size does not depend on the GPU's SM count
  int rc = sb200::can_implement(g);
  if (rc) return rc;
  if (sb200::workspace_bytes(g) > static_cast<size_t>(SB200_STATIC_SCRATCH_BYTES)) return SB200_ERR_SCRATCH_TOO_LARGE;
  void* scratch = nullptr;
  if ((rc = scratch_address(&scratch))) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // run() clears the status block at the head of the scratch on the stream before it launches; everything else
  // in the scratch (presums, hand-off tiles) is fully rewritten by the kernels before it is read.
  if ((rc = sb200::run(g, scratch, SB200_STATIC_SCRATCH_BYTES, s))) return rc;
  return wait ? sb200::read_status(scratch, s) : 0;
}
