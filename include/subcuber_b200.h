/*
 * subcuber_b200 -- C ABI of the Blackwell (sm_100a) Strassen-Winograd GEMM backend.
 *
 * Two groups of entry points:
 *
 *  1. `run_<kernel>`: the benchmark-driver ABI of the reference project.  Signature, argument meaning,
 *     ownership and error behaviour are those of `extern "C" int run_<kernel>(KernelRunnerBuffers, ...)`
 *     in the reference (src/cuda/kernel_runner.cpp:27-32, src/cuda/kernel_runner_support.cuh:16-21,48-178,
 *     544-578): a, b, d are DEVICE pointers owned by the caller, packed row-major (lda = k, ldb = n,
 *     ldd = n); c may be NULL and is never read (beta = 0); the callee allocates and frees its own
 *     workspace; D = A * B; *avg_ms is the mean over `iterations` timed runs after `warmup_iterations`
 *     untimed ones, measured with CUDA events on streams[0].  Return 0 on success; otherwise one of the
 *     SB200_ERR_* codes below (same meaning as the reference's int(cutlass::Status)), an int(cudaError_t),
 *     10000 + cublasStatus_t for the cuBLAS rows (src/cuda/cublas_runner.cpp:37-39), or a device status
 *     code >= 100 when a kernel gave up on a bounded wait.  No exception crosses the boundary.
 *     Only streams[0] is used: products that the reference spreads over 7 or 49 streams run inside one
 *     persistent kernel here.  split_k_slices must be 1.
 *
 *  2. `sb200_*`: the operator itself (one GEMM, asynchronous on a stream), for callers that manage
 *     their own buffers, and a host-buffer convenience call.
 */
#ifndef SUBCUBER_B200_H_
#define SUBCUBER_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference: src/cuda/kernel_runner_support.cuh:16-21 */
typedef struct KernelRunnerBuffers {
  const void* a;
  const void* b;
  const void* c;
  void* d;
} KernelRunnerBuffers;

/* Opaque CUDA stream handle (cudaStream_t) without requiring cuda_runtime.h in C callers. */
typedef struct CUstream_st* sb200_stream_t;

enum {
  SB200_OK = 0,
  SB200_ERR_MISALIGNED_OPERAND = 1, /* a row of an operand or quadrant does not start on 16 bytes   */
  SB200_ERR_INVALID_PROBLEM = 4,    /* non-positive or (level >= 1) odd sizes, NULL operand         */
  SB200_ERR_NOT_SUPPORTED = 5,      /* unknown kernel / dtype / split_k_slices != 1                 */
  SB200_ERR_WORKSPACE_NULL = 6,     /* workspace missing, too small or not 256-byte aligned         */
  SB200_ERR_INTERNAL = 7,
  SB200_ERR_NO_KERNEL = 8,          /* kernel name not in the registry                              */
  SB200_STATUS_PRODUCER_TIMEOUT = 101, /* device: a bounded wait gave up (role in the code)        */
  SB200_STATUS_MMA_TIMEOUT = 102,
  SB200_STATUS_EPILOGUE_TIMEOUT = 103,
  SB200_STATUS_PRESUM_TIMEOUT = 104,
  SB200_STATUS_SPLIT_TIMEOUT = 105, /* the second K-half of a split tile waited in vain for the first half's sum */
  SB200_STATUS_PEER_TIMEOUT = 201   /* sb200_peer_wait: a counter another GPU should have raised did not arrive      */
};

/* ---- group 1: kernel_runner ABI (reference: src/cuda/kernel_runner.cpp:27-32) --------------------- */
#define SB200_DECLARE_RUN(name)                                                                          \
  int name(KernelRunnerBuffers buffers, int m, int n, int k, int warmup_iterations, int iterations,    \
           sb200_stream_t* streams, int num_streams, int split_k_slices, float* avg_ms)

/* Level 0 (plain GEMM on tcgen05); registry rows analogous to the reference's *_cutlass_* kernels
 * (src/cuda/kernel_runner.cpp:127-137). */
SB200_DECLARE_RUN(run_blackwell_f16_cubic_128x256);
SB200_DECLARE_RUN(run_blackwell_f16_cubic_128x128);
SB200_DECLARE_RUN(run_blackwell_f32_cubic_128x256); /* fp32 storage, TF32 tensor-core math */
SB200_DECLARE_RUN(run_blackwell_f32_cubic_128x128);
/* Level 1, presums formed in shared memory each k-step ("FUSED_IN_SUM" variants of the reference,
 * src/cuda/kernel_runner.cpp:148,150,161,164,179). */
SB200_DECLARE_RUN(run_blackwell_f16_sw_fused_presum);
SB200_DECLARE_RUN(run_blackwell_f32_sw_fused_presum);
/* Level 1, presums written to a workspace by the launch that computes M0 and M1 ("PRESUM" /
 * interleaved variants of the reference, src/cuda/kernel_runner.cpp:140-141,144-145,151-152). */
SB200_DECLARE_RUN(run_blackwell_f16_sw_interleaved_presum);
SB200_DECLARE_RUN(run_blackwell_f32_sw_interleaved_presum);
/* CTA-pair variants: 256 x 256 tiles computed by two SMs with tcgen05.mma.cta_group::2 (each SM loads half of B). */
SB200_DECLARE_RUN(run_blackwell_f16_cubic_2sm_256x256);
SB200_DECLARE_RUN(run_blackwell_f32_cubic_2sm_256x256);
SB200_DECLARE_RUN(run_blackwell_f16_sw_fused_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_f32_sw_fused_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_f16_sw_interleaved_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_f32_sw_interleaved_presum_2sm);
/* Level 1 in ONE launch: the seven products of a tile run back to back in one CTA pair while the presum warps of the
 * same launch materialise the presums and publish them panel by panel (the reference runs several Mi in one CTA with
 * FusedMiGroup, include/cutlass/gemm/device/strassen_decls.h:1466-1539, but always launches its presum step first). */
SB200_DECLARE_RUN(run_blackwell_f16_sw_merged_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_f32_sw_merged_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_bf16_sw_merged_presum_2sm);
/* Level 2 (49 products): seven level-1 interleaved-presum groups over half-size operands, 14 launches, chained through
 * fp32 buffers.  Stands where the reference has StrassenGemmLevel2 (include/cutlass/gemm/device/strassen_gemm.h:
 * 1300-2008) behind its "*_level_2" runner entries. */
SB200_DECLARE_RUN(run_blackwell_f16_sw_level2);
SB200_DECLARE_RUN(run_blackwell_f32_sw_level2);
SB200_DECLARE_RUN(run_blackwell_f16_sw_level2_2sm);
SB200_DECLARE_RUN(run_blackwell_f32_sw_level2_2sm);
/* bfloat16 storage, fp32 accumulate: the f16 kernels with the other 16-bit format (same tiles, programs and plans; the
 * reference has no bfloat16 kernels and lists the type as future work, README.md:179). */
SB200_DECLARE_RUN(run_cublas_bf16);
SB200_DECLARE_RUN(run_blackwell_bf16_cubic_128x256);
SB200_DECLARE_RUN(run_blackwell_bf16_cubic_2sm_256x256);
SB200_DECLARE_RUN(run_blackwell_bf16_sw_fused_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_bf16_sw_interleaved_presum);
SB200_DECLARE_RUN(run_blackwell_bf16_sw_interleaved_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_bf16_sw_level2);
SB200_DECLARE_RUN(run_blackwell_bf16_sw_level2_2sm);
SB200_DECLARE_RUN(run_blackwell_bf16_sw_auto);
/* Level 1 of Strassen's original algorithm (7 products, 18 additions; no operand sums more than two blocks), one launch,
 * operand sums formed in shared memory.  The reference names other Strassen-like algorithms as future work
 * (README.md:179) and leaves StrassenType::Strassen stubbed (include/cutlass/gemm/kernel/strassen_gemm.h:1360-1398). */
SB200_DECLARE_RUN(run_blackwell_f16_strassen_fused_presum);
SB200_DECLARE_RUN(run_blackwell_f32_strassen_fused_presum);
SB200_DECLARE_RUN(run_blackwell_f16_strassen_fused_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_f32_strassen_fused_presum_2sm);
/* the same algorithm on materialised presums (a launch without products forms them, a second launch multiplies) */
SB200_DECLARE_RUN(run_blackwell_f16_strassen_presum_2sm);
SB200_DECLARE_RUN(run_blackwell_f32_strassen_presum_2sm);
/* fp64 on the double-precision tensor-core instruction (mma.sync.m16n8k16.f64): plain GEMM, level 1 (2 standalone
 * presum launches + 7 product launches whose epilogue adds the postsums) and level 2 (2 + 7 x 9 launches).  Stand where the reference has its f64 DMMA kernels
 * (src/cuda/kernels/ampere_f64_*.cu via kernel_runner.cpp:99-180). */
SB200_DECLARE_RUN(run_blackwell_f64_cubic_dmma);
SB200_DECLARE_RUN(run_blackwell_f64_sw_level1);
SB200_DECLARE_RUN(run_blackwell_f64_sw_level2);
/* Level (0, 1 or 2) and kernel family chosen by problem size, crossover points measured on B200: the role of the
 * reference front end's size-based choice (src/compile.py:200-212).  Accepted wherever a kernel name is. */
SB200_DECLARE_RUN(run_blackwell_f16_sw_auto);
SB200_DECLARE_RUN(run_blackwell_f32_sw_auto);
SB200_DECLARE_RUN(run_blackwell_f64_sw_auto);
/* Name of the kernel "blackwell_<dtype>_sw_auto" resolves to for this problem (dtype: "f16" | "bf16" | "f32" | "f64"). */
const char* sb200_auto_kernel(const char* dtype, int m, int n, int k);
/* cuBLAS baselines behind the same ABI (reference: src/cuda/cublas_runner.cpp:151-175); the tf32 row is
 * an addition: the reference's f32 row is CUBLAS_COMPUTE_32F_PEDANTIC (cublas_runner.cpp:14). */
SB200_DECLARE_RUN(run_cublas_f16);
SB200_DECLARE_RUN(run_cublas_f32);
SB200_DECLARE_RUN(run_cublas_f64);
SB200_DECLARE_RUN(run_cublas_tf32);
/* cuBLASLt baselines (reference: src/cuda/cublaslt_runner.cpp:42-272). */
SB200_DECLARE_RUN(run_cublaslt_f16);
SB200_DECLARE_RUN(run_cublaslt_f32);
SB200_DECLARE_RUN(run_cublaslt_f64);

/* Registry: the rows a driver lists (reference: `KernelEntry kKernels[]`, src/cuda/kernel_runner.cpp:99-181). */
typedef SB200_DECLARE_RUN((*sb200_run_fn));
typedef struct sb200_kernel_entry {
  const char* name;
  const char* arch;  /* "blackwell" */
  const char* dtype; /* "f16" | "bf16" | "f32" | "f64" */
  int strassen_level;
  sb200_run_fn run;
} sb200_kernel_entry;
int sb200_num_kernels(void);
const sb200_kernel_entry* sb200_kernel(int index);

/* ---- group 2: the operator (reference: device::StrassenGemm life cycle can_implement /
 *      get_workspace_size / initialize / run, include/cutlass/gemm/device/strassen_gemm.h:538-1117) -- */

/* 0 if `kernel` (a registry name without the "run_" prefix, e.g. "blackwell_f16_sw_interleaved_presum")
 * can run m x n x k, else an error code. */
int sb200_gemm_can_implement(const char* kernel, int m, int n, int k);
/* Bytes of device workspace one call needs (0 on unknown kernel). */
size_t sb200_gemm_workspace_bytes(const char* kernel, int m, int n, int k);
/* Enqueue D = A * B on `stream` (device pointers, packed row-major).  Asynchronous.  `workspace` must be
 * 256-byte aligned device memory of at least sb200_gemm_workspace_bytes().  Allocates nothing. */
int sb200_gemm(const char* kernel, const void* a, const void* b, void* d, int m, int n, int k, void* workspace,
               size_t workspace_bytes, sb200_stream_t stream);
/* Per-call options of the tensor-core kernels (f16, bf16, f32); a NULL pointer or a zeroed struct means defaults.
 * The reference's operators take their tuning through their Arguments struct in the same way (split_k_slices,
 * raster order and swizzle: src/cuda/kernel_runner_support.cuh:328,341).  The workspace size depends on sm_limit and
 * no_split (they decide which tiles are split along K), so size the workspace with the same options. */
typedef struct sb200_gemm_options {
  int sm_limit;         /* SMs the kernels may occupy; 0 = all.  A caller that overlaps its own kernels (e.g. a
                           collective) with the GEMM keeps the remaining SMs free for them */
  int no_split;         /* 1: never compute the tiles of a partial last wave as two K-halves */
  int wait_limit_us;    /* bound of every device-side wait in microseconds; 0 = 2 s */
  int drop_split_flags; /* test aid for the give-up path: the first K-halves of split tiles do not publish their flags,
                           the second halves' waits run out after wait_limit_us and the status word reads
                           SB200_STATUS_SPLIT_TIMEOUT; the output of such a call is incomplete */
} sb200_gemm_options;
size_t sb200_gemm_workspace_bytes_opt(const char* kernel, int m, int n, int k, const sb200_gemm_options* options);
int sb200_gemm_opt(const char* kernel, const void* a, const void* b, void* d, int m, int n, int k, void* workspace,
                   size_t workspace_bytes, sb200_stream_t stream, const sb200_gemm_options* options);
/* The unit list of one launch of a tensor-core kernel on a device of `sms` SMs (0 = the current device): whole output
 * tiles in raster order, then two units for each tile of a last wave that is at most half full - the tile's two
 * column halves (CTA-pair kernels: independent units, drawn with the whole tiles by whichever pair is free) or its
 * two K-halves that run at the same time (1-CTA kernels, dealt round-robin; the role the reference gives to
 * split_k_slices, src/cuda/kernel_runner.cpp:244-255).  Writes 10 ints per unit in list order: worker under a
 * round-robin deal, tile, part (0 = all of K or the K-half that publishes its partial sum, 1 = the K-half that adds
 * it), parts (1 or 2), first k-step, end k-step, hand-off slot, split slot, column half (0 or 1), column parts (1 or
 * 2).  Returns the number of units (negative: error code); *workers = CTAs or CTA pairs launched.  Host arithmetic
 * only. */
int sb200_gemm_deal(const char* kernel, int m, int n, int k, const sb200_gemm_options* options, int sms, int* units,
                    int max_units, int* workers);
/* General form D = alpha * (A * B) + beta * C (the argument set of the reference's operators,
 * include/cutlass/gemm/device/strassen_gemm.h:365-451; the reference's runner fixes alpha = 1, beta = 0).  C is m x n
 * row-major in the output type, may be the same buffer as D, and is read only when beta != 0.  The scaling is applied
 * in fp32 (fp64 for the f64 kernels) to the finished sum, once, before the rounding to the output type. */
int sb200_gemm_ex(const char* kernel, double alpha, const void* a, const void* b, double beta, const void* c, void* d,
                  int m, int n, int k, void* workspace, size_t workspace_bytes, sb200_stream_t stream);
/* Column-major A (m x k), B (k x n), D (m x n), each packed: runs the row-major kernels on the swapped problem
 * (the reference's swap trick, strassen_gemm.h:3925-4170).  Workspace size: sb200_gemm_workspace_bytes(kernel, n, m, k). */
int sb200_gemm_colmajor(const char* kernel, const void* a, const void* b, void* d, int m, int n, int k, void* workspace,
                        size_t workspace_bytes, sb200_stream_t stream);
/* Synchronise `stream` and return the device status word of the last sb200_gemm on `workspace`
 * (0 = every bounded wait was satisfied). */
int sb200_gemm_status(void* workspace, sb200_stream_t stream);
/* Kernel launches one sb200_gemm call makes for this kernel name. */
int sb200_gemm_launches(const char* kernel);
/* Host-buffer convenience: copies A and B to the device, runs, copies D back, synchronously.
 * Allocates and frees device memory inside the call. */
int sb200_gemm_host(const char* kernel, const void* a_host, const void* b_host, void* d_host, int m, int n, int k);


/* D = A * B (f16, Strassen-Winograd level 1, the "blackwell_f16_sw_interleaved_presum" kernels) for callers
 * that are not allowed to allocate device memory: a serving process whose memory pool owns the whole GPU, a
 * latency-critical loop that cannot take the device-wide synchronisation cudaMalloc/cudaFree imply, a plugin
 * host that grants libraries no allocation rights.  No counterpart in the reference project, whose operators
 * always allocate their workspace per call (src/cuda/kernel_runner_support.cuh:90-91).
 *
 * The scratch memory the kernels need lives in a fixed array of SB200_STATIC_SCRATCH_BYTES inside the library,
 * resident on every GPU that uses this call until the process exits.  The call itself performs no cudaMalloc,
 * cudaFree or other allocating call.  Limits:
 *  - the problem's scratch (sb200_gemm_workspace_bytes_opt of that kernel with no_split = 1: this call never cuts
 *    tiles along K, so that its scratch does not depend on the GPU's SM count) must fit, else SB200_ERR_SCRATCH_TOO_LARGE
 *    is returned and nothing runs (the 33 MiB of the array cover m = n = k = 2048, which needs 32 MiB and 256 bytes;
 *    2048 x 2048 x 2304 already needs 34 MiB, 3072^3 72 MiB, 4096^3 128 MiB);
 *  - one array per GPU, shared by all calls and never cleared between them except for what must start at zero
 *    (the status block, cleared on `stream` by every call): calls whose kernels could overlap on the GPU race on
 *    it, so order them on one stream (or otherwise serialise them);
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *    current) and loads the kernels: make that first call before starting any stream capture.
 * a, b, d: device pointers, packed row-major.  wait != 0: synchronise `stream` and return the device status word
 * (0 = ok); wait == 0: return after the launches are enqueued. */
#define SB200_STATIC_SCRATCH_BYTES (33u << 20)
#define SB200_ERR_SCRATCH_TOO_LARGE 9
int sb200_gemm_f16_sw_static_scratch(const void* a, const void* b, void* d, int m, int n, int k,
                                     sb200_stream_t stream, int wait);

/* Byte offsets of the parts of the workspace of (kernel, m, n, k).  presum_a holds S1,S2,A02,A1S2 packed
 * [4][mq][kq] and presum_b holds B10,B31,S3,S3B2 packed [4][kq][nq] in the operand type (interleaved-presum
 * kernels only: the counterpart of the reference's presum workspace, strassen_gemm.h:653-657); handoff[i] are
 * fp32 tile-contiguous buffers. */
typedef struct sb200_workspace_layout {
  size_t status, presum_a, presum_b, handoff[4], total;
  int mq, nq, kq, tiles_m, tiles_n, bn;
} sb200_workspace_layout;
int sb200_gemm_workspace_layout(const char* kernel, int m, int n, int k, sb200_workspace_layout* out);

/* Like sb200_gemm, but synchronises and reports the device time of each kernel launch of the call
 * (CUDA events on `stream`); launch_ms must have room for SB200_MAX_LAUNCHES floats. */
#define SB200_MAX_LAUNCHES 80
int sb200_gemm_timed(const char* kernel, const void* a, const void* b, void* d, int m, int n, int k, void* workspace,
                     size_t workspace_bytes, sb200_stream_t stream, float* launch_ms, int* num_launches);

/* Per-launch device timing inside a caller's own timed loop: sb200_gemm_events is sb200_gemm that also records
 * launches+1 CUDA events of `list`, starting at `first_index`, before the first and after every kernel launch. */
typedef struct sb200_event_list sb200_event_list;
sb200_event_list* sb200_events_create(int count);
void sb200_events_destroy(sb200_event_list* list);
int sb200_events_elapsed_ms(sb200_event_list* list, int first, int second, float* ms);
int sb200_gemm_events(const char* kernel, const void* a, const void* b, void* d, int m, int n, int k, void* workspace,
                      size_t workspace_bytes, sb200_stream_t stream, sb200_event_list* list, int first_index,
                      const sb200_gemm_options* options);

/* The tile program tables the kernels interpret (csrc/tile_program.h), for inspection and tests.
 * which: "level0" | "level1_full_fly" | "level1_full_ws" | "level1_first" | "level1_first_early" | "level1_second" |
 * "level1_second_taps" |
 * "level2_<child>_launch<1|2>" with child in m0, m1, m2, m4, m5, m3, m6. */
int sb200_tile_program(const char* which, void* out, size_t out_bytes);
size_t sb200_tile_program_bytes(void);

/* ---- flags between the GPUs of one box (the multi-GPU plan's operand exchange; the reference is single-GPU,
 *      src/cuda/kernel_runner_support.cuh:312, and has no counterpart) ----------------------------------------------
 * The exchange moves operand shards with the copy engines; these two calls order it.  A flag is a 32-bit counter in
 * the receiving GPU's memory; the sender reaches it through a peer mapping (plain stores over NVLink).
 * sb200_peer_signal enqueues a one-block kernel that stores `value` (release, system scope) to each of `count` flag
 * addresses; behind copies on the same stream it announces that they have landed.  sb200_peer_wait enqueues a
 * one-block kernel that waits until each of `count` local flags is >= `value`; the wait is bounded (wait_limit_us
 * microseconds, 0 = 2 s): when it runs out the kernel stores SB200_STATUS_PEER_TIMEOUT to *status (a device int the
 * caller zeroed) and returns, so a peer that never arrives cannot hang this GPU. */
#define SB200_MAX_PEERS 16
int sb200_peer_signal(int* const* peer_flags, int count, int value, sb200_stream_t stream);
int sb200_peer_wait(int* const* local_flags, int count, int value, unsigned wait_limit_us, int* status,
                    sb200_stream_t stream);

/* Seeded synthetic inputs, bit-identical on host and device for dist 0 and 2 (dist 1 uses libm / device
 * math and agrees to rounding).  dtype: 0 f16, 1 f32, 2 f64, 3 bf16.  dist: 0 uniform[-1,1), 1 normal(0,1),
 * 2 the reference harness' value set (multiples of 0.25 in [-4,4] for f16, [-16,16] otherwise;
 * tests/base_test.cuh:248-262 in the reference).  Element i takes Philox4x32-10(key = seed,
 * counter = (i, subsequence)); by convention A uses subsequence 0 and B subsequence 1. */
int sb200_fill_device(int dtype, int dist, unsigned long long seed, unsigned subsequence, void* device_ptr,
                      unsigned long long count, sb200_stream_t stream);
int sb200_fill_host(int dtype, int dist, unsigned long long seed, unsigned subsequence, void* host_ptr,
                    unsigned long long count);

#ifdef __cplusplus
}
#endif
#endif /* SUBCUBER_B200_H_ */
