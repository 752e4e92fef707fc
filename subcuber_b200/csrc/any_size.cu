// Entry points of the host-side operator for every problem size: problems the kernels take as they are go straight to
// the tensor-core path (sw_host.cu) or the fp64 path (dgemm_sw.cu); the rest run on zero-padded copies of the operands
// held behind the kernels' own workspace.  The reference operators reject such problems
// (include/cutlass/gemm/device/strassen_gemm.h:484-507 can_implement: alignment and tile-multiple checks); its general
// GEMM form D = alpha * A * B + beta * C (:365-451) is kept on the padded path by padding C into the padded output.
#include <stdint.h>
#include <string.h>

#include "sw_host.h"

namespace sb200 {
namespace {

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int esize_of(DType t) { return (t == kF16 || t == kBF16) ? 2 : (t == kF32 ? 4 : 8); }
inline int level_of(Variant v) { return v == kCubic ? 0 : (v == kInterleavedLevel2 ? 2 : 1); }

struct PadPlan {
  bool needed;
  int mp, np, kp;                       // padded extents
  size_t inner, off_a, off_b, off_d, total;  // workspace: [kernels' own workspace][A'][B'][D']
};

int inner_can_implement(const GemmArgs& a) { return a.dtype == kF64 ? f64::can_implement(a) : tc::can_implement(a); }
size_t inner_workspace(const GemmArgs& a) { return a.dtype == kF64 ? f64::workspace_bytes(a) : tc::workspace_bytes(a); }
int inner_launches(const GemmArgs& a) { return a.dtype == kF64 ? f64::launches_per_run(a) : tc::launches_per_run(a); }

// The padded problem with its operands in the workspace at `base` (base == nullptr: addresses stand for alignment
// only, for the checks and the size).
GemmArgs padded_args(const GemmArgs& a, const PadPlan& p, char* base) {
  GemmArgs g = a;
  char* b = base ? base : reinterpret_cast<char*>(uintptr_t(256));
  g.m = p.mp; g.n = p.np; g.k = p.kp;
  g.a = b + p.off_a;
  g.b = b + p.off_b;
  g.d = b + p.off_d;
  g.c = (a.scaled && a.beta != 0.0) ? g.d : nullptr;
  g.events = nullptr;
  return g;
}

PadPlan plan(const GemmArgs& a) {
  PadPlan p;
  memset(&p, 0, sizeof(p));
  p.mp = a.m; p.np = a.n; p.kp = a.k;
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return p;
  const int es = esize_of(a.dtype);
  const int vec = 16 / es;
  if (a.dtype == kF64) {
    // the fp64 kernels want extents that divide into blocks whose rows are 16-byte aligned
    const int div = 1 << level_of(a.variant);
    p.mp = static_cast<int>(align_up(a.m, div));
    p.np = static_cast<int>(align_up(a.n, size_t(div) * vec));
    p.kp = static_cast<int>(align_up(a.k, size_t(div) * vec));
  } else {
    // the tensor-core kernels want 16-byte aligned rows only
    p.np = static_cast<int>(align_up(a.n, vec));
    p.kp = static_cast<int>(align_up(a.k, vec));
  }
  p.needed = p.mp != a.m || p.np != a.n || p.kp != a.k;
  if (!p.needed) return p;
  p.off_a = 0;
  p.off_b = align_up(p.off_a + size_t(p.mp) * p.kp * es, 256);
  p.off_d = align_up(p.off_b + size_t(p.kp) * p.np * es, 256);
  p.total = align_up(p.off_d + size_t(p.mp) * p.np * es, 256);
  p.inner = align_up(inner_workspace(padded_args(a, p, nullptr)), 256);
  p.off_a += p.inner; p.off_b += p.inner; p.off_d += p.inner;
  p.total += p.inner;
  return p;
}

// dst (rows_d x cols_d, packed, cols_d a multiple of 16 bytes) = src (rows_s x cols_s, leading dimension ld_s) in its
// top-left corner, zeros elsewhere.  Each thread gathers 16 bytes of a destination row element by element (the source
// needs no more than element alignment) and stores them at once.
template <typename T>
__global__ void pad_copy_kernel(T* __restrict__ dst, int rows_d, int cols_d, const T* __restrict__ src, int rows_s,
                                int cols_s, long long ld_s) {
  constexpr int V = 16 / sizeof(T);
  const int vec_per_row = cols_d / V;
  const long long total = static_cast<long long>(rows_d) * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / vec_per_row);
    const int c0 = static_cast<int>(i - static_cast<long long>(r) * vec_per_row) * V;
    alignas(16) T tmp[V];
#pragma unroll
    for (int e = 0; e < V; ++e) tmp[e] = (r < rows_s && c0 + e < cols_s) ? src[r * ld_s + c0 + e] : T(0);
    *reinterpret_cast<uint4*>(dst + static_cast<long long>(r) * cols_d + c0) = *reinterpret_cast<const uint4*>(tmp);
  }
}

// dst (rows x cols, leading dimension ld_d) = top-left corner of src (packed, cols_s columns, a multiple of 16 bytes):
// 16 bytes read at once, written element by element.
template <typename T>
__global__ void crop_copy_kernel(T* __restrict__ dst, long long ld_d, int rows, int cols, const T* __restrict__ src,
                                 int cols_s) {
  constexpr int V = 16 / sizeof(T);
  const int vec_per_row = (cols + V - 1) / V;
  const long long total = static_cast<long long>(rows) * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / vec_per_row);
    const int c0 = static_cast<int>(i - static_cast<long long>(r) * vec_per_row) * V;
    alignas(16) T tmp[V];
    *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(src + static_cast<long long>(r) * cols_s + c0);
#pragma unroll
    for (int e = 0; e < V; ++e)
      if (c0 + e < cols) dst[r * ld_d + c0 + e] = tmp[e];
  }
}

int copy_grid(long long elements) {
  const long long blocks = (elements / 4 + 255) / 256;  // a thread moves 16 bytes (2 to 8 elements) per iteration
  return static_cast<int>(blocks < 148 * 16 ? (blocks < 1 ? 1 : blocks) : 148 * 16);
}

template <typename T>
int pad_copy(void* dst, int rows_d, int cols_d, const void* src, int rows_s, int cols_s, long long ld_s,
             cudaStream_t stream) {
  pad_copy_kernel<T><<<copy_grid(static_cast<long long>(rows_d) * cols_d), 256, 0, stream>>>(
      static_cast<T*>(dst), rows_d, cols_d, static_cast<const T*>(src), rows_s, cols_s, ld_s);
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int crop_copy(void* dst, long long ld_d, int rows, int cols, const void* src, int cols_s, cudaStream_t stream) {
  crop_copy_kernel<T><<<copy_grid(static_cast<long long>(rows) * cols), 256, 0, stream>>>(
      static_cast<T*>(dst), ld_d, rows, cols, static_cast<const T*>(src), cols_s);
  return static_cast<int>(cudaGetLastError());
}

int pad_copy_es(int es, void* dst, int rows_d, int cols_d, const void* src, int rows_s, int cols_s, long long ld_s,
                cudaStream_t stream) {
  if (es == 2) return pad_copy<unsigned short>(dst, rows_d, cols_d, src, rows_s, cols_s, ld_s, stream);
  if (es == 4) return pad_copy<unsigned int>(dst, rows_d, cols_d, src, rows_s, cols_s, ld_s, stream);
  return pad_copy<unsigned long long>(dst, rows_d, cols_d, src, rows_s, cols_s, ld_s, stream);
}

}  // namespace

int can_implement(const GemmArgs& a) {
  if (a.m <= 0 || a.n <= 0 || a.k <= 0 || !a.a || !a.b || !a.d) return kErrInvalidProblem;
  if (a.dtype != kF16 && a.dtype != kF32 && a.dtype != kF64 && a.dtype != kBF16) return kErrNotSupported;
  if (a.scaled && a.beta != 0.0 && !a.c) return kErrInvalidProblem;
  const PadPlan p = plan(a);
  return p.needed ? inner_can_implement(padded_args(a, p, nullptr)) : inner_can_implement(a);
}

size_t workspace_bytes(const GemmArgs& a) {
  const PadPlan p = plan(a);
  return p.needed ? p.total : inner_workspace(a);
}

WorkspaceLayout workspace_layout(const GemmArgs& a) {
  const PadPlan p = plan(a);
  const GemmArgs g = p.needed ? padded_args(a, p, nullptr) : a;
  WorkspaceLayout w;
  if (g.dtype == kF64) {
    memset(&w, 0, sizeof(w));
  } else {
    w = tc::workspace_layout(g);
  }
  w.total = workspace_bytes(a);
  return w;
}

int launches_per_run(const GemmArgs& a) {
  const PadPlan p = plan(a);
  if (!p.needed) return inner_launches(a);
  // copies of A and B (and C when it is read), the kernels, the copy of D
  return 2 + ((a.scaled && a.beta != 0.0) ? 1 : 0) + inner_launches(padded_args(a, p, nullptr)) + 1;
}

int run(const GemmArgs& a, void* workspace, size_t workspace_size, cudaStream_t stream) {
  int rc = can_implement(a);
  if (rc) return rc;
  const PadPlan p = plan(a);
  if (!p.needed) return a.dtype == kF64 ? f64::run(a, workspace, workspace_size, stream) : tc::run(a, workspace, workspace_size, stream);
  if (!workspace || workspace_size < p.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return kErrWorkspaceNull;
  const int es = esize_of(a.dtype);
  GemmArgs g = padded_args(a, p, static_cast<char*>(workspace));
  int nev = 0;
  auto mark = [&]() -> int { return a.events ? static_cast<int>(cudaEventRecord(a.events[nev++], stream)) : 0; };
  if ((rc = mark())) return rc;
  if ((rc = pad_copy_es(es, const_cast<void*>(g.a), p.mp, p.kp, a.a, a.m, a.k, a.k, stream))) return rc;
  if ((rc = mark())) return rc;
  if ((rc = pad_copy_es(es, const_cast<void*>(g.b), p.kp, p.np, a.b, a.k, a.n, a.n, stream))) return rc;
  if ((rc = mark())) return rc;
  if (g.c) {
    if ((rc = pad_copy_es(es, g.d, p.mp, p.np, a.c, a.m, a.n, a.n, stream))) return rc;
    if ((rc = mark())) return rc;
  }
  // the kernels' events continue the list: their first event is the one just recorded
  if (a.events) g.events = a.events + (nev - 1);
  rc = a.dtype == kF64 ? f64::run(g, workspace, p.inner, stream) : tc::run(g, workspace, p.inner, stream);
  if (rc) return rc;
  nev += inner_launches(g);
  if (es == 2) rc = crop_copy<unsigned short>(a.d, a.n, a.m, a.n, g.d, p.np, stream);
  else if (es == 4) rc = crop_copy<unsigned int>(a.d, a.n, a.m, a.n, g.d, p.np, stream);
  else rc = crop_copy<unsigned long long>(a.d, a.n, a.m, a.n, g.d, p.np, stream);
  if (rc) return rc;
  return mark();
}

}  // namespace sb200
