// State that belongs to one device of the process (a kernel's shared-memory attribute, the SM count) is kept per
// device ordinal: a process may drive several GPUs, and host threads may call concurrently.
#pragma once
#include <cuda_runtime.h>

#include <atomic>

namespace sb200 {

constexpr int kMaxDevices = 64;

// One flag per device ordinal.  `run_once` calls `set()` (e.g. cudaFuncSetAttribute, which applies to the current
// device's copy of a kernel) the first time it is reached with a given device current.  Two threads that race on the
// same device may both call `set()`: the calls are idempotent, so that is harmless.
struct PerDeviceOnce {
  std::atomic<unsigned long long> done{0};
  template <typename SetFn>
  int run_once(SetFn set) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    const bool tracked = dev >= 0 && dev < kMaxDevices;
    const unsigned long long bit = tracked ? (1ull << dev) : 0ull;
    if (tracked && (done.load(std::memory_order_acquire) & bit)) return 0;
    const int rc = set();
    if (rc == 0 && tracked) done.fetch_or(bit, std::memory_order_release);
    return rc;
  }
};

// SM count of the current device (0 when it cannot be read).
inline int sm_count_of_current_device() {
  static std::atomic<int> cache[kMaxDevices];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  const bool tracked = dev >= 0 && dev < kMaxDevices;
  if (tracked) {
    const int c = cache[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (tracked) cache[dev].store(n, std::memory_order_relaxed);
  return n;
}

}  // namespace sb200
