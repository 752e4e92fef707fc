// extern "C" boundary of the library: the reference benchmark driver's `run_<kernel>` entry points
// (src/cuda/kernel_runner.cpp:27-32 in the reference project), the kernel registry and the `sb200_*` operator calls.
#include <cublasLt.h>
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <string.h>

#include "../../include/subcuber_b200.h"
#include "sw_host.h"
#include "sw_programs.h"

namespace {

using sb200::DType;
using sb200::GemmArgs;
using sb200::Variant;

struct KernelDesc {
  const char* name;
  const char* dtype;
  int level;
  DType dt;
  Variant variant;
  int bn;
  int pair;
};

const KernelDesc kDescs[] = {
    {"blackwell_f16_cubic_128x256", "f16", 0, sb200::kF16, sb200::kCubic, 256, 0},
    {"blackwell_f16_cubic_128x128", "f16", 0, sb200::kF16, sb200::kCubic, 128, 0},
    {"blackwell_f32_cubic_128x256", "f32", 0, sb200::kF32, sb200::kCubic, 256, 0},
    {"blackwell_f32_cubic_128x128", "f32", 0, sb200::kF32, sb200::kCubic, 128, 0},
    {"blackwell_f16_sw_fused_presum", "f16", 1, sb200::kF16, sb200::kFusedPresum, 256, 0},
    {"blackwell_f32_sw_fused_presum", "f32", 1, sb200::kF32, sb200::kFusedPresum, 256, 0},
    {"blackwell_f16_sw_interleaved_presum", "f16", 1, sb200::kF16, sb200::kInterleavedPresum, 256, 0},
    {"blackwell_f32_sw_interleaved_presum", "f32", 1, sb200::kF32, sb200::kInterleavedPresum, 256, 0},
    {"blackwell_f16_cubic_2sm_256x256", "f16", 0, sb200::kF16, sb200::kCubic, 256, 1},
    {"blackwell_f32_cubic_2sm_256x256", "f32", 0, sb200::kF32, sb200::kCubic, 256, 1},
    {"blackwell_f16_sw_fused_presum_2sm", "f16", 1, sb200::kF16, sb200::kFusedPresum, 256, 1},
    {"blackwell_f32_sw_fused_presum_2sm", "f32", 1, sb200::kF32, sb200::kFusedPresum, 256, 1},
    {"blackwell_f16_sw_interleaved_presum_2sm", "f16", 1, sb200::kF16, sb200::kInterleavedPresum, 256, 1},
    {"blackwell_f32_sw_interleaved_presum_2sm", "f32", 1, sb200::kF32, sb200::kInterleavedPresum, 256, 1},
    {"blackwell_f16_sw_merged_presum_2sm", "f16", 1, sb200::kF16, sb200::kMergedPresum, 256, 1},
    {"blackwell_f32_sw_merged_presum_2sm", "f32", 1, sb200::kF32, sb200::kMergedPresum, 256, 1},
    {"blackwell_bf16_sw_merged_presum_2sm", "bf16", 1, sb200::kBF16, sb200::kMergedPresum, 256, 1},
    {"blackwell_f16_sw_level2", "f16", 2, sb200::kF16, sb200::kInterleavedLevel2, 256, 0},
    {"blackwell_f32_sw_level2", "f32", 2, sb200::kF32, sb200::kInterleavedLevel2, 256, 0},
    {"blackwell_f16_sw_level2_2sm", "f16", 2, sb200::kF16, sb200::kInterleavedLevel2, 256, 1},
    {"blackwell_f32_sw_level2_2sm", "f32", 2, sb200::kF32, sb200::kInterleavedLevel2, 256, 1},
    {"blackwell_bf16_cubic_128x256", "bf16", 0, sb200::kBF16, sb200::kCubic, 256, 0},
    {"blackwell_bf16_cubic_2sm_256x256", "bf16", 0, sb200::kBF16, sb200::kCubic, 256, 1},
    {"blackwell_bf16_sw_fused_presum_2sm", "bf16", 1, sb200::kBF16, sb200::kFusedPresum, 256, 1},
    {"blackwell_bf16_sw_interleaved_presum", "bf16", 1, sb200::kBF16, sb200::kInterleavedPresum, 256, 0},
    {"blackwell_bf16_sw_interleaved_presum_2sm", "bf16", 1, sb200::kBF16, sb200::kInterleavedPresum, 256, 1},
    {"blackwell_bf16_sw_level2", "bf16", 2, sb200::kBF16, sb200::kInterleavedLevel2, 256, 0},
    {"blackwell_bf16_sw_level2_2sm", "bf16", 2, sb200::kBF16, sb200::kInterleavedLevel2, 256, 1},
    {"blackwell_f16_strassen_fused_presum", "f16", 1, sb200::kF16, sb200::kStrassenFused, 256, 0},
    {"blackwell_f32_strassen_fused_presum", "f32", 1, sb200::kF32, sb200::kStrassenFused, 256, 0},
    {"blackwell_f16_strassen_fused_presum_2sm", "f16", 1, sb200::kF16, sb200::kStrassenFused, 256, 1},
    {"blackwell_f32_strassen_fused_presum_2sm", "f32", 1, sb200::kF32, sb200::kStrassenFused, 256, 1},
    {"blackwell_f16_strassen_presum_2sm", "f16", 1, sb200::kF16, sb200::kStrassenPresum, 256, 1},
    {"blackwell_f32_strassen_presum_2sm", "f32", 1, sb200::kF32, sb200::kStrassenPresum, 256, 1},
    {"blackwell_f64_cubic_dmma", "f64", 0, sb200::kF64, sb200::kCubic, 0, 0},
    {"blackwell_f64_sw_level1", "f64", 1, sb200::kF64, sb200::kFusedPresum, 0, 0},
    {"blackwell_f64_sw_level2", "f64", 2, sb200::kF64, sb200::kInterleavedLevel2, 0, 0},
};
constexpr int kNumDescs = sizeof(kDescs) / sizeof(kDescs[0]);

const KernelDesc* find_desc(const char* name) {
  if (!name) return nullptr;
  for (int i = 0; i < kNumDescs; ++i)
    if (strcmp(kDescs[i].name, name) == 0) return &kDescs[i];
  return nullptr;
}

// Size-based choice of level and kernel family ("blackwell_<dtype>_sw_auto"): the role of the reference front end's
// cost model (src/compile.py:200-212, should_use_k2 / level by size), with crossover points measured on B200.
// The recursion pays off once a product is large enough for its presum and postsum traffic to be small against it:
//   f16 : level 1 from 12288, level 2 from 24576 (smallest of m, n, k); below that the plain pair kernel is fastest
//   bf16: the same kernels with the other 16-bit format, the same crossover points
//   tf32: level 1 from 12288, level 2 from 16384
//   f64 : level 1 from 6144, level 2 from 16384
const char* auto_kernel(sb200::DType dt, int m, int n, int k) {
  int s = m < n ? m : n;
  if (k < s) s = k;
  switch (dt) {
    case sb200::kF16:
      if (s >= 24576) return "blackwell_f16_sw_level2_2sm";
      if (s >= 12288) return "blackwell_f16_sw_interleaved_presum_2sm";
      return "blackwell_f16_cubic_2sm_256x256";
    case sb200::kBF16:
      if (s >= 24576) return "blackwell_bf16_sw_level2_2sm";
      if (s >= 12288) return "blackwell_bf16_sw_interleaved_presum_2sm";
      return "blackwell_bf16_cubic_2sm_256x256";
    case sb200::kF32:
      if (s >= 16384) return "blackwell_f32_sw_level2_2sm";
      if (s >= 12288) return "blackwell_f32_sw_interleaved_presum_2sm";
      return "blackwell_f32_cubic_2sm_256x256";
    default:
      if (s >= 16384) return "blackwell_f64_sw_level2";
      if (s >= 6144) return "blackwell_f64_sw_level1";
      return "blackwell_f64_cubic_dmma";
  }
}

// Registry name -> descriptor for a given problem: "…_sw_auto" names resolve by size, all others by name.
const KernelDesc* resolve_desc(const char* name, int m, int n, int k) {
  if (!name) return nullptr;
  if (strcmp(name, "blackwell_f16_sw_auto") == 0) return find_desc(auto_kernel(sb200::kF16, m, n, k));
  if (strcmp(name, "blackwell_bf16_sw_auto") == 0) return find_desc(auto_kernel(sb200::kBF16, m, n, k));
  if (strcmp(name, "blackwell_f32_sw_auto") == 0) return find_desc(auto_kernel(sb200::kF32, m, n, k));
  if (strcmp(name, "blackwell_f64_sw_auto") == 0) return find_desc(auto_kernel(sb200::kF64, m, n, k));
  return find_desc(name);
}

GemmArgs make_args(const KernelDesc& d, const void* a, const void* b, void* out, int m, int n, int k,
                   const sb200_gemm_options* opt = nullptr) {
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.dtype = d.dt;
  g.variant = d.variant;
  g.m = m;
  g.n = n;
  g.k = k;
  g.a = a;
  g.b = b;
  g.d = out;
  g.bn = d.bn;
  g.pair = d.pair;
  g.sm_limit = 0;
  if (opt) {
    g.sm_limit = opt->sm_limit > 0 ? opt->sm_limit : 0;
    g.no_split = opt->no_split != 0;
    g.wait_limit_us = opt->wait_limit_us > 0 ? opt->wait_limit_us : 0;
    g.drop_split_flags = opt->drop_split_flags != 0;
  }
  return g;
}

// Timing harness of one registry row: the shape of kernel_runner_run_cutlass2 in the reference
// (src/cuda/kernel_runner_support.cuh:48-178): check, allocate workspace, warm up, time `iterations` runs with
// CUDA events, free.  Events are recorded on the stream the kernels run on.
int run_registry_kernel(const char* name, KernelRunnerBuffers buf, int m, int n, int k, int warmup, int iterations,
                        sb200_stream_t* streams, int num_streams, int split_k, float* avg_ms) {
  const KernelDesc* d = resolve_desc(name, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  if (split_k != 1) return SB200_ERR_NOT_SUPPORTED;
  if (iterations <= 0 || warmup < 0 || !avg_ms) return SB200_ERR_INVALID_PROBLEM;
  GemmArgs g = make_args(*d, buf.a, buf.b, buf.d, m, n, k);
  int rc = sb200::can_implement(g);
  if (rc) return rc;
  cudaStream_t stream = (streams && num_streams > 0) ? reinterpret_cast<cudaStream_t>(streams[0]) : nullptr;
  const size_t ws_bytes = sb200::workspace_bytes(g);
  void* ws = nullptr;
  cudaError_t ce = cudaMalloc(&ws, ws_bytes);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  cudaEvent_t start = nullptr, stop = nullptr;
  auto cleanup = [&]() {
    if (start) cudaEventDestroy(start);
    if (stop) cudaEventDestroy(stop);
    cudaFree(ws);
  };
  for (int i = 0; i < warmup; ++i) {
    rc = sb200::run(g, ws, ws_bytes, stream);
    if (rc) { cleanup(); return rc; }
  }
  rc = sb200::read_status(ws, stream);
  if (rc) { cleanup(); return rc; }
  if ((ce = cudaEventCreate(&start)) != cudaSuccess || (ce = cudaEventCreate(&stop)) != cudaSuccess ||
      (ce = cudaEventRecord(start, stream)) != cudaSuccess) {
    cleanup();
    return static_cast<int>(ce);
  }
  for (int i = 0; i < iterations; ++i) {
    rc = sb200::run(g, ws, ws_bytes, stream);
    if (rc) { cleanup(); return rc; }
  }
  if ((ce = cudaEventRecord(stop, stream)) != cudaSuccess || (ce = cudaEventSynchronize(stop)) != cudaSuccess) {
    cleanup();
    return static_cast<int>(ce);
  }
  float ms = 0.f;
  if ((ce = cudaEventElapsedTime(&ms, start, stop)) != cudaSuccess) { cleanup(); return static_cast<int>(ce); }
  rc = sb200::read_status(ws, stream);
  cleanup();
  if (rc) return rc;
  *avg_ms = ms / static_cast<float>(iterations);
  return 0;
}

// ------------------------------------------------------------------------------------------- cuBLAS rows
int cublas_err(cublasStatus_t s) { return s == CUBLAS_STATUS_SUCCESS ? 0 : 10000 + static_cast<int>(s); }

struct BlasType {
  cudaDataType_t data;
  cublasComputeType_t compute;
  cublasMath_t math;
  cublasGemmAlgo_t algo;
  bool f64;
};
// f16 / f32 / f64 rows use the reference's settings (src/cuda/cublas_runner.cpp:9-35).
const BlasType kBlasF16 = {CUDA_R_16F, CUBLAS_COMPUTE_32F_FAST_16F, CUBLAS_TENSOR_OP_MATH, CUBLAS_GEMM_DEFAULT_TENSOR_OP, false};
const BlasType kBlasBF16 = {CUDA_R_16BF, CUBLAS_COMPUTE_32F, CUBLAS_TENSOR_OP_MATH, CUBLAS_GEMM_DEFAULT_TENSOR_OP, false};
const BlasType kBlasF32 = {CUDA_R_32F, CUBLAS_COMPUTE_32F_PEDANTIC, CUBLAS_DEFAULT_MATH, CUBLAS_GEMM_DEFAULT, false};
const BlasType kBlasF64 = {CUDA_R_64F, CUBLAS_COMPUTE_64F_PEDANTIC, CUBLAS_DEFAULT_MATH, CUBLAS_GEMM_DEFAULT, true};
const BlasType kBlasTF32 = {CUDA_R_32F, CUBLAS_COMPUTE_32F_FAST_TF32, CUBLAS_TF32_TENSOR_OP_MATH, CUBLAS_GEMM_DEFAULT_TENSOR_OP, false};

template <typename Launch>
int time_launches(Launch launch, cudaStream_t stream, int warmup, int iterations, float* avg_ms) {
  int rc;
  for (int i = 0; i < warmup; ++i)
    if ((rc = launch())) return rc;
  cudaError_t ce = cudaStreamSynchronize(stream);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  cudaEvent_t start = nullptr, stop = nullptr;
  if ((ce = cudaEventCreate(&start)) != cudaSuccess) return static_cast<int>(ce);
  if ((ce = cudaEventCreate(&stop)) != cudaSuccess) { cudaEventDestroy(start); return static_cast<int>(ce); }
  auto done = [&](int code) { cudaEventDestroy(start); cudaEventDestroy(stop); return code; };
  if ((ce = cudaEventRecord(start, stream)) != cudaSuccess) return done(static_cast<int>(ce));
  for (int i = 0; i < iterations; ++i)
    if ((rc = launch())) return done(rc);
  if ((ce = cudaEventRecord(stop, stream)) != cudaSuccess) return done(static_cast<int>(ce));
  if ((ce = cudaEventSynchronize(stop)) != cudaSuccess) return done(static_cast<int>(ce));
  float ms = 0.f;
  if ((ce = cudaEventElapsedTime(&ms, start, stop)) != cudaSuccess) return done(static_cast<int>(ce));
  *avg_ms = ms / static_cast<float>(iterations);
  return done(0);
}

// Row-major D = A * B through column-major cuBLAS by swapping the operands
// (reference: src/cuda/cublas_runner.cpp:81-90).
int run_cublas(const BlasType& t, KernelRunnerBuffers buf, int m, int n, int k, int warmup, int iterations,
               sb200_stream_t* streams, int num_streams, float* avg_ms) {
  if (m <= 0 || n <= 0 || k <= 0 || iterations <= 0 || warmup < 0 || !avg_ms) return SB200_ERR_INVALID_PROBLEM;
  cudaStream_t stream = (streams && num_streams > 0) ? reinterpret_cast<cudaStream_t>(streams[0]) : nullptr;
  cublasHandle_t h = nullptr;
  cublasStatus_t s = cublasCreate(&h);
  if (s != CUBLAS_STATUS_SUCCESS) return cublas_err(s);
  int rc = 0;
  if ((s = cublasSetStream(h, stream)) != CUBLAS_STATUS_SUCCESS || (s = cublasSetMathMode(h, t.math)) != CUBLAS_STATUS_SUCCESS) {
    cublasDestroy(h);
    return cublas_err(s);
  }
  float alpha_f = 1.f, beta_f = 0.f;
  double alpha_d = 1.0, beta_d = 0.0;
  const void* alpha = t.f64 ? static_cast<const void*>(&alpha_d) : static_cast<const void*>(&alpha_f);
  const void* beta = t.f64 ? static_cast<const void*>(&beta_d) : static_cast<const void*>(&beta_f);
  auto launch = [&]() {
    return cublas_err(cublasGemmEx(h, CUBLAS_OP_N, CUBLAS_OP_N, n, m, k, alpha, buf.b, t.data, n, buf.a, t.data, k, beta,
                                   buf.d, t.data, n, t.compute, t.algo));
  };
  rc = time_launches(launch, stream, warmup, iterations, avg_ms);
  cublasDestroy(h);
  return rc;
}

// cuBLASLt with row-order layouts, one heuristic result and a 32 MiB workspace
// (reference: src/cuda/cublaslt_runner.cpp:59,74-187).
int run_cublaslt(const BlasType& t, KernelRunnerBuffers buf, int m, int n, int k, int warmup, int iterations,
                 sb200_stream_t* streams, int num_streams, float* avg_ms) {
  if (m <= 0 || n <= 0 || k <= 0 || iterations <= 0 || warmup < 0 || !avg_ms) return SB200_ERR_INVALID_PROBLEM;
  cudaStream_t stream = (streams && num_streams > 0) ? reinterpret_cast<cudaStream_t>(streams[0]) : nullptr;
  cublasLtHandle_t h = nullptr;
  cublasLtMatmulDesc_t desc = nullptr;
  cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
  cublasLtMatmulPreference_t pref = nullptr;
  void* ws = nullptr;
  const size_t ws_bytes = size_t(32) << 20;
  auto cleanup = [&]() {
    if (ws) cudaFree(ws);
    if (pref) cublasLtMatmulPreferenceDestroy(pref);
    if (lc) cublasLtMatrixLayoutDestroy(lc);
    if (lb) cublasLtMatrixLayoutDestroy(lb);
    if (la) cublasLtMatrixLayoutDestroy(la);
    if (desc) cublasLtMatmulDescDestroy(desc);
    if (h) cublasLtDestroy(h);
  };
  cublasStatus_t s;
#define LT_CHECK(call)                      \
  if ((s = (call)) != CUBLAS_STATUS_SUCCESS) { \
    cleanup();                              \
    return cublas_err(s);                   \
  }
  LT_CHECK(cublasLtCreate(&h));
  LT_CHECK(cublasLtMatmulDescCreate(&desc, t.compute, t.f64 ? CUDA_R_64F : CUDA_R_32F));
  cublasOperation_t op = CUBLAS_OP_N;
  LT_CHECK(cublasLtMatmulDescSetAttribute(desc, CUBLASLT_MATMUL_DESC_TRANSA, &op, sizeof(op)));
  LT_CHECK(cublasLtMatmulDescSetAttribute(desc, CUBLASLT_MATMUL_DESC_TRANSB, &op, sizeof(op)));
  LT_CHECK(cublasLtMatrixLayoutCreate(&la, t.data, m, k, k));
  LT_CHECK(cublasLtMatrixLayoutCreate(&lb, t.data, k, n, n));
  LT_CHECK(cublasLtMatrixLayoutCreate(&lc, t.data, m, n, n));
  cublasLtOrder_t order = CUBLASLT_ORDER_ROW;
  LT_CHECK(cublasLtMatrixLayoutSetAttribute(la, CUBLASLT_MATRIX_LAYOUT_ORDER, &order, sizeof(order)));
  LT_CHECK(cublasLtMatrixLayoutSetAttribute(lb, CUBLASLT_MATRIX_LAYOUT_ORDER, &order, sizeof(order)));
  LT_CHECK(cublasLtMatrixLayoutSetAttribute(lc, CUBLASLT_MATRIX_LAYOUT_ORDER, &order, sizeof(order)));
  LT_CHECK(cublasLtMatmulPreferenceCreate(&pref));
  LT_CHECK(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws_bytes, sizeof(ws_bytes)));
  cudaError_t ce = cudaMalloc(&ws, ws_bytes);
  if (ce != cudaSuccess) { cleanup(); return static_cast<int>(ce); }
  cublasLtMatmulHeuristicResult_t heur;
  memset(&heur, 0, sizeof(heur));
  int found = 0;
  LT_CHECK(cublasLtMatmulAlgoGetHeuristic(h, desc, la, lb, lc, lc, pref, 1, &heur, &found));
  if (found == 0) { cleanup(); return cublas_err(CUBLAS_STATUS_NOT_SUPPORTED); }
#undef LT_CHECK
  float alpha_f = 1.f, beta_f = 0.f;
  double alpha_d = 1.0, beta_d = 0.0;
  const void* alpha = t.f64 ? static_cast<const void*>(&alpha_d) : static_cast<const void*>(&alpha_f);
  const void* beta = t.f64 ? static_cast<const void*>(&beta_d) : static_cast<const void*>(&beta_f);
  auto launch = [&]() {
    return cublas_err(cublasLtMatmul(h, desc, alpha, buf.a, la, buf.b, lb, beta, buf.d, lc, buf.d, lc, &heur.algo, ws,
                                     ws_bytes, stream));
  };
  int rc = time_launches(launch, stream, warmup, iterations, avg_ms);
  cleanup();
  return rc;
}

}  // namespace

// ------------------------------------------------------------------------------------------- exports
#define SB200_DEFINE_RUN(kernel)                                                                              \
  extern "C" int run_##kernel(KernelRunnerBuffers buffers, int m, int n, int k, int warmup_iterations,        \
                              int iterations, sb200_stream_t* streams, int num_streams, int split_k_slices,   \
                              float* avg_ms) {                                                                \
    return run_registry_kernel(#kernel, buffers, m, n, k, warmup_iterations, iterations, streams, num_streams, \
                               split_k_slices, avg_ms);                                                       \
  }

SB200_DEFINE_RUN(blackwell_f16_cubic_128x256)
SB200_DEFINE_RUN(blackwell_f16_cubic_128x128)
SB200_DEFINE_RUN(blackwell_f32_cubic_128x256)
SB200_DEFINE_RUN(blackwell_f32_cubic_128x128)
SB200_DEFINE_RUN(blackwell_f16_sw_fused_presum)
SB200_DEFINE_RUN(blackwell_f32_sw_fused_presum)
SB200_DEFINE_RUN(blackwell_f16_sw_interleaved_presum)
SB200_DEFINE_RUN(blackwell_f32_sw_interleaved_presum)
SB200_DEFINE_RUN(blackwell_f16_cubic_2sm_256x256)
SB200_DEFINE_RUN(blackwell_f32_cubic_2sm_256x256)
SB200_DEFINE_RUN(blackwell_f16_sw_fused_presum_2sm)
SB200_DEFINE_RUN(blackwell_f32_sw_fused_presum_2sm)
SB200_DEFINE_RUN(blackwell_f16_sw_interleaved_presum_2sm)
SB200_DEFINE_RUN(blackwell_f32_sw_interleaved_presum_2sm)
SB200_DEFINE_RUN(blackwell_f16_sw_merged_presum_2sm)
SB200_DEFINE_RUN(blackwell_f32_sw_merged_presum_2sm)
SB200_DEFINE_RUN(blackwell_bf16_sw_merged_presum_2sm)
SB200_DEFINE_RUN(blackwell_f16_sw_level2)
SB200_DEFINE_RUN(blackwell_f32_sw_level2)
SB200_DEFINE_RUN(blackwell_f16_sw_level2_2sm)
SB200_DEFINE_RUN(blackwell_f32_sw_level2_2sm)
SB200_DEFINE_RUN(blackwell_bf16_cubic_128x256)
SB200_DEFINE_RUN(blackwell_bf16_cubic_2sm_256x256)
SB200_DEFINE_RUN(blackwell_bf16_sw_fused_presum_2sm)
SB200_DEFINE_RUN(blackwell_bf16_sw_interleaved_presum)
SB200_DEFINE_RUN(blackwell_bf16_sw_interleaved_presum_2sm)
SB200_DEFINE_RUN(blackwell_bf16_sw_level2)
SB200_DEFINE_RUN(blackwell_bf16_sw_level2_2sm)
SB200_DEFINE_RUN(blackwell_bf16_sw_auto)
SB200_DEFINE_RUN(blackwell_f16_strassen_fused_presum)
SB200_DEFINE_RUN(blackwell_f32_strassen_fused_presum)
SB200_DEFINE_RUN(blackwell_f16_strassen_fused_presum_2sm)
SB200_DEFINE_RUN(blackwell_f32_strassen_fused_presum_2sm)
SB200_DEFINE_RUN(blackwell_f16_strassen_presum_2sm)
SB200_DEFINE_RUN(blackwell_f32_strassen_presum_2sm)
SB200_DEFINE_RUN(blackwell_f64_cubic_dmma)
SB200_DEFINE_RUN(blackwell_f64_sw_level1)
SB200_DEFINE_RUN(blackwell_f64_sw_level2)
SB200_DEFINE_RUN(blackwell_f16_sw_auto)
SB200_DEFINE_RUN(blackwell_f32_sw_auto)
SB200_DEFINE_RUN(blackwell_f64_sw_auto)

#define SB200_DEFINE_BLAS(fn, impl, type)                                                                      \
  extern "C" int fn(KernelRunnerBuffers buffers, int m, int n, int k, int warmup_iterations, int iterations,   \
                    sb200_stream_t* streams, int num_streams, int, float* avg_ms) {                            \
    return impl(type, buffers, m, n, k, warmup_iterations, iterations, streams, num_streams, avg_ms);          \
  }
SB200_DEFINE_BLAS(run_cublas_f16, run_cublas, kBlasF16)
SB200_DEFINE_BLAS(run_cublas_bf16, run_cublas, kBlasBF16)
SB200_DEFINE_BLAS(run_cublas_f32, run_cublas, kBlasF32)
SB200_DEFINE_BLAS(run_cublas_f64, run_cublas, kBlasF64)
SB200_DEFINE_BLAS(run_cublas_tf32, run_cublas, kBlasTF32)
SB200_DEFINE_BLAS(run_cublaslt_f16, run_cublaslt, kBlasF16)
SB200_DEFINE_BLAS(run_cublaslt_f32, run_cublaslt, kBlasF32)
SB200_DEFINE_BLAS(run_cublaslt_f64, run_cublaslt, kBlasF64)

static const sb200_kernel_entry kRegistry[] = {
    {"cublas_f32", "blackwell", "f32", 0, run_cublas_f32},
    {"cublas_f16", "blackwell", "f16", 0, run_cublas_f16},
    {"cublas_f64", "blackwell", "f64", 0, run_cublas_f64},
    {"cublas_tf32", "blackwell", "f32", 0, run_cublas_tf32},
    {"cublas_bf16", "blackwell", "bf16", 0, run_cublas_bf16},
    {"cublaslt_f32", "blackwell", "f32", 0, run_cublaslt_f32},
    {"cublaslt_f16", "blackwell", "f16", 0, run_cublaslt_f16},
    {"cublaslt_f64", "blackwell", "f64", 0, run_cublaslt_f64},
    {"blackwell_f16_cubic_128x256", "blackwell", "f16", 0, run_blackwell_f16_cubic_128x256},
    {"blackwell_f16_cubic_128x128", "blackwell", "f16", 0, run_blackwell_f16_cubic_128x128},
    {"blackwell_f32_cubic_128x256", "blackwell", "f32", 0, run_blackwell_f32_cubic_128x256},
    {"blackwell_f32_cubic_128x128", "blackwell", "f32", 0, run_blackwell_f32_cubic_128x128},
    {"blackwell_f16_sw_fused_presum", "blackwell", "f16", 1, run_blackwell_f16_sw_fused_presum},
    {"blackwell_f32_sw_fused_presum", "blackwell", "f32", 1, run_blackwell_f32_sw_fused_presum},
    {"blackwell_f16_sw_interleaved_presum", "blackwell", "f16", 1, run_blackwell_f16_sw_interleaved_presum},
    {"blackwell_f32_sw_interleaved_presum", "blackwell", "f32", 1, run_blackwell_f32_sw_interleaved_presum},
    {"blackwell_f16_cubic_2sm_256x256", "blackwell", "f16", 0, run_blackwell_f16_cubic_2sm_256x256},
    {"blackwell_f32_cubic_2sm_256x256", "blackwell", "f32", 0, run_blackwell_f32_cubic_2sm_256x256},
    {"blackwell_f16_sw_fused_presum_2sm", "blackwell", "f16", 1, run_blackwell_f16_sw_fused_presum_2sm},
    {"blackwell_f32_sw_fused_presum_2sm", "blackwell", "f32", 1, run_blackwell_f32_sw_fused_presum_2sm},
    {"blackwell_f16_sw_interleaved_presum_2sm", "blackwell", "f16", 1, run_blackwell_f16_sw_interleaved_presum_2sm},
    {"blackwell_f32_sw_interleaved_presum_2sm", "blackwell", "f32", 1, run_blackwell_f32_sw_interleaved_presum_2sm},
    {"blackwell_f16_sw_merged_presum_2sm", "blackwell", "f16", 1, run_blackwell_f16_sw_merged_presum_2sm},
    {"blackwell_f32_sw_merged_presum_2sm", "blackwell", "f32", 1, run_blackwell_f32_sw_merged_presum_2sm},
    {"blackwell_bf16_sw_merged_presum_2sm", "blackwell", "bf16", 1, run_blackwell_bf16_sw_merged_presum_2sm},
    {"blackwell_f16_sw_level2", "blackwell", "f16", 2, run_blackwell_f16_sw_level2},
    {"blackwell_f32_sw_level2", "blackwell", "f32", 2, run_blackwell_f32_sw_level2},
    {"blackwell_f16_sw_level2_2sm", "blackwell", "f16", 2, run_blackwell_f16_sw_level2_2sm},
    {"blackwell_f32_sw_level2_2sm", "blackwell", "f32", 2, run_blackwell_f32_sw_level2_2sm},
    {"blackwell_bf16_cubic_128x256", "blackwell", "bf16", 0, run_blackwell_bf16_cubic_128x256},
    {"blackwell_bf16_cubic_2sm_256x256", "blackwell", "bf16", 0, run_blackwell_bf16_cubic_2sm_256x256},
    {"blackwell_bf16_sw_fused_presum_2sm", "blackwell", "bf16", 1, run_blackwell_bf16_sw_fused_presum_2sm},
    {"blackwell_bf16_sw_interleaved_presum", "blackwell", "bf16", 1, run_blackwell_bf16_sw_interleaved_presum},
    {"blackwell_bf16_sw_interleaved_presum_2sm", "blackwell", "bf16", 1, run_blackwell_bf16_sw_interleaved_presum_2sm},
    {"blackwell_bf16_sw_level2", "blackwell", "bf16", 2, run_blackwell_bf16_sw_level2},
    {"blackwell_bf16_sw_level2_2sm", "blackwell", "bf16", 2, run_blackwell_bf16_sw_level2_2sm},
    {"blackwell_f16_strassen_fused_presum", "blackwell", "f16", 1, run_blackwell_f16_strassen_fused_presum},
    {"blackwell_f32_strassen_fused_presum", "blackwell", "f32", 1, run_blackwell_f32_strassen_fused_presum},
    {"blackwell_f16_strassen_fused_presum_2sm", "blackwell", "f16", 1, run_blackwell_f16_strassen_fused_presum_2sm},
    {"blackwell_f32_strassen_fused_presum_2sm", "blackwell", "f32", 1, run_blackwell_f32_strassen_fused_presum_2sm},
    {"blackwell_f16_strassen_presum_2sm", "blackwell", "f16", 1, run_blackwell_f16_strassen_presum_2sm},
    {"blackwell_f32_strassen_presum_2sm", "blackwell", "f32", 1, run_blackwell_f32_strassen_presum_2sm},
    {"blackwell_f64_cubic_dmma", "blackwell", "f64", 0, run_blackwell_f64_cubic_dmma},
    {"blackwell_f64_sw_level1", "blackwell", "f64", 1, run_blackwell_f64_sw_level1},
    {"blackwell_f64_sw_level2", "blackwell", "f64", 2, run_blackwell_f64_sw_level2},
    // level chosen by size; listed under level 1 so that "--strassen_level=1" runs show it next to the fixed plans
    {"blackwell_f16_sw_auto", "blackwell", "f16", 1, run_blackwell_f16_sw_auto},
    {"blackwell_bf16_sw_auto", "blackwell", "bf16", 1, run_blackwell_bf16_sw_auto},
    {"blackwell_f32_sw_auto", "blackwell", "f32", 1, run_blackwell_f32_sw_auto},
    {"blackwell_f64_sw_auto", "blackwell", "f64", 1, run_blackwell_f64_sw_auto},
};

extern "C" int sb200_num_kernels(void) { return static_cast<int>(sizeof(kRegistry) / sizeof(kRegistry[0])); }
extern "C" const sb200_kernel_entry* sb200_kernel(int index) {
  return (index >= 0 && index < sb200_num_kernels()) ? &kRegistry[index] : nullptr;
}

extern "C" int sb200_gemm_can_implement(const char* kernel, int m, int n, int k) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  // operand pointers are checked by sb200_gemm; use aligned placeholders here
  GemmArgs g = make_args(*d, reinterpret_cast<const void*>(256), reinterpret_cast<const void*>(256),
                         reinterpret_cast<void*>(256), m, n, k);
  return sb200::can_implement(g);
}

extern "C" size_t sb200_gemm_workspace_bytes(const char* kernel, int m, int n, int k) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d || m <= 0 || n <= 0 || k <= 0) return 0;
  GemmArgs g = make_args(*d, nullptr, nullptr, nullptr, m, n, k);
  return sb200::workspace_bytes(g);
}

extern "C" int sb200_gemm(const char* kernel, const void* a, const void* b, void* d_out, int m, int n, int k,
                          void* workspace, size_t workspace_bytes, sb200_stream_t stream) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  GemmArgs g = make_args(*d, a, b, d_out, m, n, k);
  return sb200::run(g, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" size_t sb200_gemm_workspace_bytes_opt(const char* kernel, int m, int n, int k,
                                                 const sb200_gemm_options* options) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d || m <= 0 || n <= 0 || k <= 0) return 0;
  GemmArgs g = make_args(*d, nullptr, nullptr, nullptr, m, n, k, options);
  return sb200::workspace_bytes(g);
}

extern "C" int sb200_gemm_deal(const char* kernel, int m, int n, int k, const sb200_gemm_options* options, int sms,
                               int* units, int max_units, int* workers) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return -SB200_ERR_NO_KERNEL;
  if (!units || max_units < 0 || m <= 0 || n <= 0 || k <= 0 || d->dt == sb200::kF64) return -SB200_ERR_INVALID_PROBLEM;
  GemmArgs g = make_args(*d, nullptr, nullptr, nullptr, m, n, k, options);
  return sb200::tc::deal_units(g, sms, units, max_units, workers);
}

extern "C" int sb200_gemm_opt(const char* kernel, const void* a, const void* b, void* d_out, int m, int n, int k,
                              void* workspace, size_t workspace_bytes, sb200_stream_t stream,
                              const sb200_gemm_options* options) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  GemmArgs g = make_args(*d, a, b, d_out, m, n, k, options);
  return sb200::run(g, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int sb200_gemm_ex(const char* kernel, double alpha, const void* a, const void* b, double beta, const void* c,
                             void* d_out, int m, int n, int k, void* workspace, size_t workspace_bytes,
                             sb200_stream_t stream) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  GemmArgs g = make_args(*d, a, b, d_out, m, n, k);
  g.scaled = 1;
  g.alpha = alpha;
  g.beta = beta;
  g.c = c;
  return sb200::run(g, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

// Column-major operands: the same memory read row-major holds the transposes, and (A B)^T = B^T A^T, so the
// row-major kernels run with the operands swapped (the reference's swap trick,
// include/cutlass/gemm/device/strassen_gemm.h:3925-4170).
extern "C" int sb200_gemm_colmajor(const char* kernel, const void* a, const void* b, void* d_out, int m, int n, int k,
                                   void* workspace, size_t workspace_bytes, sb200_stream_t stream) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  GemmArgs g = make_args(*d, b, a, d_out, n, m, k);
  return sb200::run(g, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" const char* sb200_auto_kernel(const char* dtype, int m, int n, int k) {
  if (!dtype) return nullptr;
  if (strcmp(dtype, "f16") == 0) return auto_kernel(sb200::kF16, m, n, k);
  if (strcmp(dtype, "bf16") == 0) return auto_kernel(sb200::kBF16, m, n, k);
  if (strcmp(dtype, "f32") == 0) return auto_kernel(sb200::kF32, m, n, k);
  if (strcmp(dtype, "f64") == 0) return auto_kernel(sb200::kF64, m, n, k);
  return nullptr;
}

extern "C" int sb200_gemm_status(void* workspace, sb200_stream_t stream) {
  if (!workspace) return SB200_ERR_WORKSPACE_NULL;
  return sb200::read_status(workspace, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int sb200_gemm_launches(const char* kernel) {
  const KernelDesc* d = find_desc(kernel);
  if (!d) return 0;
  GemmArgs g = make_args(*d, nullptr, nullptr, nullptr, 1024, 1024, 1024);  // a problem the kernels take as it is
  return sb200::launches_per_run(g);
}

extern "C" int sb200_gemm_host(const char* kernel, const void* a_host, const void* b_host, void* d_host, int m, int n,
                               int k) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  if (!a_host || !b_host || !d_host || m <= 0 || n <= 0 || k <= 0) return SB200_ERR_INVALID_PROBLEM;
  const size_t es = (d->dt == sb200::kF16 || d->dt == sb200::kBF16) ? 2 : (d->dt == sb200::kF64 ? 8 : 4);
  const size_t a_bytes = size_t(m) * k * es, b_bytes = size_t(k) * n * es, d_bytes = size_t(m) * n * es;
  void *da = nullptr, *db = nullptr, *dd = nullptr, *ws = nullptr;
  int rc = 0;
  cudaError_t ce = cudaSuccess;
  auto cleanup = [&]() { cudaFree(da); cudaFree(db); cudaFree(dd); cudaFree(ws); };
  if ((ce = cudaMalloc(&da, a_bytes)) != cudaSuccess || (ce = cudaMalloc(&db, b_bytes)) != cudaSuccess ||
      (ce = cudaMalloc(&dd, d_bytes)) != cudaSuccess) {
    cleanup();
    return static_cast<int>(ce);
  }
  GemmArgs g = make_args(*d, da, db, dd, m, n, k);
  if ((rc = sb200::can_implement(g))) { cleanup(); return rc; }
  const size_t ws_bytes = sb200::workspace_bytes(g);
  if ((ce = cudaMalloc(&ws, ws_bytes)) != cudaSuccess) { cleanup(); return static_cast<int>(ce); }
  if ((ce = cudaMemcpyAsync(da, a_host, a_bytes, cudaMemcpyHostToDevice, nullptr)) != cudaSuccess ||
      (ce = cudaMemcpyAsync(db, b_host, b_bytes, cudaMemcpyHostToDevice, nullptr)) != cudaSuccess) {
    cleanup();
    return static_cast<int>(ce);
  }
  if ((rc = sb200::run(g, ws, ws_bytes, nullptr))) { cleanup(); return rc; }
  if ((ce = cudaMemcpyAsync(d_host, dd, d_bytes, cudaMemcpyDeviceToHost, nullptr)) != cudaSuccess) {
    cleanup();
    return static_cast<int>(ce);
  }
  rc = sb200::read_status(ws, nullptr);
  cleanup();
  return rc;
}

extern "C" int sb200_gemm_workspace_layout(const char* kernel, int m, int n, int k, sb200_workspace_layout* out) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  if (!out || m <= 0 || n <= 0 || k <= 0) return SB200_ERR_INVALID_PROBLEM;
  GemmArgs g = make_args(*d, nullptr, nullptr, nullptr, m, n, k);
  const sb200::WorkspaceLayout w = sb200::workspace_layout(g);
  out->status = w.status;
  out->presum_a = w.presum_a;
  out->presum_b = w.presum_b;
  for (int i = 0; i < 4; ++i) out->handoff[i] = w.handoff[i];
  out->total = w.total;
  out->mq = w.mq; out->nq = w.nq; out->kq = w.kq;
  out->tiles_m = w.tiles_m; out->tiles_n = w.tiles_n; out->bn = w.bn;
  return 0;
}

extern "C" int sb200_gemm_timed(const char* kernel, const void* a, const void* b, void* d_out, int m, int n, int k,
                                void* workspace, size_t workspace_bytes, sb200_stream_t stream, float* launch_ms,
                                int* num_launches) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  if (!launch_ms || !num_launches) return SB200_ERR_INVALID_PROBLEM;
  GemmArgs g = make_args(*d, a, b, d_out, m, n, k);
  const int nl = sb200::launches_per_run(g);
  cudaEvent_t ev[SB200_MAX_LAUNCHES + 1];
  memset(ev, 0, sizeof(ev));
  if (nl > SB200_MAX_LAUNCHES) return SB200_ERR_INTERNAL;
  cudaError_t ce = cudaSuccess;
  for (int i = 0; i <= nl; ++i)
    if ((ce = cudaEventCreate(&ev[i])) != cudaSuccess) break;
  int rc = static_cast<int>(ce);
  if (!rc) {
    g.events = ev;
    rc = sb200::run(g, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
  }
  if (!rc) rc = sb200::read_status(workspace, reinterpret_cast<cudaStream_t>(stream));
  if (!rc) {
    for (int i = 0; i < nl; ++i)
      if ((ce = cudaEventElapsedTime(&launch_ms[i], ev[i], ev[i + 1])) != cudaSuccess) rc = static_cast<int>(ce);
    *num_launches = nl;
  }
  for (int i = 0; i <= SB200_MAX_LAUNCHES; ++i)
    if (ev[i]) cudaEventDestroy(ev[i]);
  return rc;
}

extern "C" int sb200_tile_program(const char* which, void* out, size_t out_bytes) {
  if (!which || !out || out_bytes < sizeof(sb200_program_t)) return SB200_ERR_INVALID_PROBLEM;
  sb200_program_t pg;
  if (!sb200::programs::find(which, &pg)) return SB200_ERR_NO_KERNEL;
  memcpy(out, &pg, sizeof(pg));
  return 0;
}

extern "C" size_t sb200_tile_program_bytes(void) { return sizeof(sb200_program_t); }

// ---- event lists: per-launch device timing inside a caller's timed loop -------------------------------
struct sb200_event_list {
  int count;
  cudaEvent_t* ev;
};

extern "C" sb200_event_list* sb200_events_create(int count) {
  if (count <= 0) return nullptr;
  sb200_event_list* l = new sb200_event_list;
  l->count = count;
  l->ev = new cudaEvent_t[count];
  for (int i = 0; i < count; ++i) {
    if (cudaEventCreate(&l->ev[i]) != cudaSuccess) {
      for (int j = 0; j < i; ++j) cudaEventDestroy(l->ev[j]);
      delete[] l->ev;
      delete l;
      return nullptr;
    }
  }
  return l;
}

extern "C" void sb200_events_destroy(sb200_event_list* l) {
  if (!l) return;
  for (int i = 0; i < l->count; ++i) cudaEventDestroy(l->ev[i]);
  delete[] l->ev;
  delete l;
}

extern "C" int sb200_events_elapsed_ms(sb200_event_list* l, int first, int second, float* ms) {
  if (!l || !ms || first < 0 || second < 0 || first >= l->count || second >= l->count) return SB200_ERR_INVALID_PROBLEM;
  return static_cast<int>(cudaEventElapsedTime(ms, l->ev[first], l->ev[second]));
}

extern "C" int sb200_gemm_events(const char* kernel, const void* a, const void* b, void* d_out, int m, int n, int k,
                                 void* workspace, size_t workspace_bytes, sb200_stream_t stream, sb200_event_list* l,
                                 int first_index, const sb200_gemm_options* options) {
  const KernelDesc* d = resolve_desc(kernel, m, n, k);
  if (!d) return SB200_ERR_NO_KERNEL;
  GemmArgs g = make_args(*d, a, b, d_out, m, n, k, options);
  if (!l || first_index < 0 || first_index + sb200::launches_per_run(g) + 1 > l->count) return SB200_ERR_INVALID_PROBLEM;
  g.events = l->ev + first_index;
  return sb200::run(g, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}
