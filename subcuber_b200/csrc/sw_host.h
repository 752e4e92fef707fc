// Host-side operator for the Blackwell Strassen-Winograd GEMM path: argument checks, workspace carving,
// tensor-map construction and launches.  It stands where the reference project has its device-level
// operators (include/cutlass/gemm/device/strassen_gemm.h:277-1217 `StrassenGemm`: can_implement /
// get_workspace_size / initialize / run) and mirrors their four-step life cycle.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace sb200 {

// kF32: fp32 storage, TF32 tensor-core math, fp32 accumulate; kBF16: bfloat16 storage, fp32 accumulate (the f16 kernels
// with the other 16-bit format: same tiles, same programs, one run-time flag)
enum DType { kF16 = 0, kF32 = 1, kF64 = 2, kBF16 = 3 };

enum Variant {
  kCubic = 0,             // level 0, plain GEMM
  kFusedPresum = 1,       // level 1, one launch, presums formed in shared memory by the presum warps
  kInterleavedPresum = 2, // level 1, two launches, presums materialised by the first launch's presum warps
  kInterleavedLevel2 = 3, // level 2, seven level-1 interleaved groups (14 launches) chained through fp32 buffers
  kStrassenFused = 4,     // level 1 of Strassen's original algorithm, one launch, operand sums formed in shared memory
  kMergedPresum = 5,      // level 1, ONE launch: presums materialised by the launch's presum warps and published panel
                          // by panel to the products that read them (CTA-pair kernels only)
  kStrassenPresum = 6,    // level 1 of Strassen's original algorithm, two launches: its ten presums materialised by
                          // the presum warps of a launch without products, then all seven products (CTA pairs only)
};

// Error codes returned across the C ABI.  Small values keep the meaning of the reference's
// `int(cutlass::Status)` returns (kernel_runner_support.cuh:44-46); CUDA errors are passed through as
// `int(cudaError_t)` exactly as the reference does (:107,116); device-side status codes are >= 100.
enum Error {
  kOk = 0,
  kErrMisalignedOperand = 1,
  kErrInvalidProblem = 4,
  kErrNotSupported = 5,
  kErrWorkspaceNull = 6,
  kErrInternal = 7,
};

struct GemmArgs {
  DType dtype;
  Variant variant;
  int m, n, k;
  const void* a;  // m x k row-major, lda = k
  const void* b;  // k x n row-major, ldb = n
  void* d;        // m x n row-major, ldd = n;  D = A * B
  int bn;         // tile width: 256 (default when 0) or 128
  int pair;       // 1: CTA-pair kernels (256 x 256 tiles on two SMs, cta_group::2); requires bn == 256
  int sm_limit;   // SMs the kernels may occupy (0: every SM of the current device)
  int no_split;   // 1: never compute the tiles of a partial last wave as two K-halves
  int wait_limit_us;     // bound of every device-side wait in microseconds (0: 2 s)
  int drop_split_flags;  // test aid for the give-up path: the first K-halves of split tiles do not publish their
                         // flags, so the second halves' bounded waits run out and the call reports status 105
  cudaEvent_t* events;  // optional: launches_per_run()+1 events, recorded before the first and after each launch
  // D = alpha * (A * B) + beta * C when `scaled` is set (else alpha = 1, beta = 0 and `c` is never read), the general
  // form of the reference's operators (include/cutlass/gemm/device/strassen_gemm.h:365-451).  C is m x n row-major,
  // ldc = n, in the output type, and may be the same buffer as D; it is read only when beta != 0.
  int scaled;
  double alpha, beta;
  const void* c;
};

// Byte offsets of the parts of the workspace (tests read the presum buffers through this).
struct WorkspaceLayout {
  size_t status, presum_a, presum_b, handoff[4], total;
  int mq, nq, kq, tiles_m, tiles_n, bn;
};
WorkspaceLayout workspace_layout(const GemmArgs& args);

// 0 when the kernels can run this problem, else an Error.
int can_implement(const GemmArgs& args);
// Bytes of device workspace `run` needs (status word, presum buffers, fp32 hand-off tiles).
size_t workspace_bytes(const GemmArgs& args);
// Enqueue the GEMM on `stream`.  `workspace` must hold workspace_bytes(args) and be 256-byte aligned.
// Asynchronous: returns launch errors only; device-side aborts are read with `read_status`.
int run(const GemmArgs& args, void* workspace, size_t workspace_size, cudaStream_t stream);
// Synchronises `stream` and returns the device status word of the last `run` on that workspace.
int read_status(void* workspace, cudaStream_t stream);
// Launches of this library's kernels made by the last `run` with these args (for launch accounting).
int launches_per_run(const GemmArgs& args);

// The calls above accept every positive m, n, k.  Problems the kernels cannot take as they are (row pitches that are
// not multiples of 16 bytes, fp64 extents that do not divide) run on
// zero-padded copies of the operands held in the workspace (any_size.cu): the padded product equals the product, and
// the result is copied back without another rounding.
//
// Tensor-core path for f16 and f32/tf32 (sw_host.cu): same calls on problems whose rows are 16-byte aligned; extents
// that do not divide by the number of blocks leave the last block row / column short.
namespace tc {
int can_implement(const GemmArgs& args);
size_t workspace_bytes(const GemmArgs& args);
WorkspaceLayout workspace_layout(const GemmArgs& args);
int run(const GemmArgs& args, void* workspace, size_t workspace_size, cudaStream_t stream);
int launches_per_run(const GemmArgs& args);
// The unit list of one launch on a device of `sms` SMs (0: the current device): writes 8 ints per unit (worker under
// the round-robin deal, tile, part, parts, k0, k1, hand-off slot, split slot) in list order, returns the number of
// units and the worker count.  Host arithmetic only (tests read the plan through this).
int deal_units(const GemmArgs& args, int sms, int* out, int max_units, int* workers);
}  // namespace tc

// fp64 path (dgemm_sw.cu): DMMA kernels, same four calls.
//   kCubic = one launch, kFusedPresum = level 1 (2 presum + 7 product launches),
//   kInterleavedLevel2 = level 2 (2 outer presum launches + 7 x (2 + 7))
namespace f64 {
int can_implement(const GemmArgs& args);
size_t workspace_bytes(const GemmArgs& args);
int run(const GemmArgs& args, void* workspace, size_t workspace_size, cudaStream_t stream);
int launches_per_run(const GemmArgs& args);
}  // namespace f64

}  // namespace sb200
