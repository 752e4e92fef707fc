// Host drivers placed BEHIND the reference project's oracle kernel templates (see oracle/Makefile).
// TEST INFRASTRUCTURE ONLY.  Each driver replays the kernel's one-thread-per-output-element grid
// (launch geometry of src/cuda/cubic_reference.cuh:62-70 and src/cuda/strassen_reference_l1.cuh:241-248)
// as a host loop with blockDim = (1,1,1), so thread (i,j) of the device grid becomes iteration (i,j).
#pragma once

typedef _Float16 ref_half;
typedef __bf16 ref_bf16;

// rows [ref_row_begin, ref_row_end) of the thread grid are replayed (whole grid by default); a bounded row
// range is what the benchmark's CPU-reference arm times, since every output element is an independent thread.
static int ref_row_begin = 0, ref_row_end = -1;

template <typename F>
static void ref_for_each_element(int M, int N, F body) {
  const int i0 = ref_row_begin, i1 = (ref_row_end < 0 || ref_row_end > M) ? M : ref_row_end;
  const long long first = (long long)i0 * N, last = (long long)i1 * N;
#pragma omp parallel for schedule(dynamic, 64)
  for (long long e = first; e < last; ++e) {
    blockDim.x = blockDim.y = blockDim.z = 1;
    threadIdx.x = threadIdx.y = threadIdx.z = 0;
    blockIdx.x = (unsigned)(e / N);
    blockIdx.y = (unsigned)(e % N);
    body();
  }
}

template <typename TIn, typename TOut, typename TAcc>
static void ref_run(int level, int M, int N, int K, double alpha, const void *A, int lda, const void *B, int ldb,
                    double beta, void *C, int ldc) {
  const TIn *a = static_cast<const TIn *>(A);
  const TIn *b = static_cast<const TIn *>(B);
  TOut *c = static_cast<TOut *>(C);
  // dispatch rule of ReferenceStrassenWinogradGemm, src/cuda/strassen_reference_l1.cuh:236-239
  if (level != 1 || (M % 2) || (N % 2) || (K % 2)) {
    ref_for_each_element(M, N, [&] {
      ReferenceGemm_kernel<TIn, TIn, TOut, TAcc, TAcc>(M, N, K, TAcc(alpha), a, lda, b, ldb, TAcc(beta), c, ldc);
    });
  } else {
    ref_for_each_element(M, N, [&] {
      ReferenceStrassenWinogradGemm_kernel<TIn, TIn, TOut, TAcc, TAcc>(M, N, K, TAcc(alpha), a, lda, b, ldb,
                                                                        TAcc(beta), c, ldc);
    });
  }
}

// dtype: 0 = <half,half,half,float,float> (the harness instantiation, tests/base_test.cuh:290),
//        1 = all float, 2 = all double, 4 = <bfloat16,bfloat16,bfloat16,float,float> (the same templates with the
//        storage type exchanged; code 3 is the oracle's TF32 model, which the reference does not have).
extern "C" int ref_sw_gemm(int dtype, int level, int M, int N, int K, double alpha, const void *A, int lda,
                           const void *B, int ldb, double beta, void *C, int ldc) {
  if (M <= 0 || N <= 0 || K <= 0 || !A || !B || !C) return 1;
  switch (dtype) {
    case 0: ref_run<ref_half, ref_half, float>(level, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc); return 0;
    case 1: ref_run<float, float, float>(level, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc); return 0;
    case 2: ref_run<double, double, double>(level, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc); return 0;
    case 4: ref_run<ref_bf16, ref_bf16, float>(level, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc); return 0;
  }
  return 1;
}

// Same, restricted to C rows [row_begin, row_end): the other rows of C are left untouched.
extern "C" int ref_sw_gemm_rows(int dtype, int level, int M, int N, int K, double alpha, const void *A, int lda,
                                const void *B, int ldb, double beta, void *C, int ldc, int row_begin, int row_end) {
  if (row_begin < 0 || row_end > M || row_begin >= row_end) return 1;
  ref_row_begin = row_begin;
  ref_row_end = row_end;
  int rc = ref_sw_gemm(dtype, level, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  ref_row_begin = 0;
  ref_row_end = -1;
  return rc;
}

// The reference's presum dump (src/cuda/strassen_reference_l1.cuh:119-183) for ONE output column pair
// would be O(M*N*K) memory; its values do not depend on which (i, j) thread writes them beyond the
// quadrant row/column, so the driver runs threads (i, j, k) over the quadrant-sized grid
// i in [0,M/2), j in [0,N/2) only for j == 0 (A-side sums) and i == 0 (B-side sums) and repacks them into
// pa[4][M/2][K/2] = S1,S2,A02,A1S2 and pb[4][K/2][N/2] = B10,B31,S3,S3B2 (operand type).
template <typename T>
static void ref_presums_t(int M, int N, int K, const T *A, int lda, const T *B, int ldb, T *pa, T *pb) {
  int hm = M / 2, hn = N / 2, hk = K / 2;
  size_t qa = (size_t)hm * hk, qb = (size_t)hk * hn;
  // the kernel indexes sums[((i*N + j)*half_k + k)*8 + s]; give it a scratch row for one (i,j) at a time
  T *scratch = new T[(size_t)hk * 8];
  blockDim.x = blockDim.y = blockDim.z = 1;
  threadIdx.x = threadIdx.y = threadIdx.z = 0;
  for (int i = 0; i < hm; ++i) {
    for (int k = 0; k < hk; ++k) {
      blockIdx.x = (unsigned)i; blockIdx.y = 0; blockIdx.z = (unsigned)k;
      // offset of (i, j=0, k) inside the kernel's dump is (i*N*hk + k)*8; rebase so it lands in scratch
      T *base = scratch - (size_t)i * N * hk * 8;
      ReferenceStrassenWinogradPresums_kernel<T, T, T>(M, N, K, A, lda, B, ldb, base);
      size_t o = (size_t)i * hk + k;
      pa[0 * qa + o] = scratch[(size_t)k * 8 + 0];
      pa[1 * qa + o] = scratch[(size_t)k * 8 + 1];
      pa[2 * qa + o] = scratch[(size_t)k * 8 + 5];
      pa[3 * qa + o] = scratch[(size_t)k * 8 + 6];
    }
  }
  for (int j = 0; j < hn; ++j) {
    for (int k = 0; k < hk; ++k) {
      blockIdx.x = 0; blockIdx.y = (unsigned)j; blockIdx.z = (unsigned)k;
      T *base = scratch - (size_t)j * hk * 8;
      ReferenceStrassenWinogradPresums_kernel<T, T, T>(M, N, K, A, lda, B, ldb, base);
      size_t o = (size_t)k * hn + j;
      pb[0 * qb + o] = scratch[(size_t)k * 8 + 2];
      pb[1 * qb + o] = scratch[(size_t)k * 8 + 3];
      pb[2 * qb + o] = scratch[(size_t)k * 8 + 4];
      pb[3 * qb + o] = scratch[(size_t)k * 8 + 7];
    }
  }
  delete[] scratch;
}

extern "C" int ref_sw_presums(int dtype, int M, int N, int K, const void *A, int lda, const void *B, int ldb,
                              void *pa, void *pb) {
  if ((M % 2) || (N % 2) || (K % 2) || !A || !B || !pa || !pb) return 1;
  switch (dtype) {
    case 0:
      ref_presums_t<ref_half>(M, N, K, (const ref_half *)A, lda, (const ref_half *)B, ldb, (ref_half *)pa,
                              (ref_half *)pb);
      return 0;
    case 1:
      ref_presums_t<float>(M, N, K, (const float *)A, lda, (const float *)B, ldb, (float *)pa, (float *)pb);
      return 0;
    case 2:
      ref_presums_t<double>(M, N, K, (const double *)A, lda, (const double *)B, ldb, (double *)pa, (double *)pb);
      return 0;
  }
  return 1;
}
