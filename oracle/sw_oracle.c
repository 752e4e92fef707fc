/*
 * CPU oracle for the Strassen-Winograd GEMM path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference project's own test oracle.
 * It is never linked into, imported by, or called from the shipped library; only
 * the tests, the smoke check and the CPU-baseline leg of the benchmark use it, and
 * only as the checker.
 *
 * What each routine follows (paths inside the reference project):
 *   orc_gemm      src/cuda/cubic_reference.cuh:10-40        naive GEMM, one accumulator per C element,
 *                                                           k ascending, D = alpha*acc + beta*C
 *   orc_sw_presums src/cuda/strassen_reference_l1.cuh:55-85 the eight operand combinations, formed in the
 *                                                           accumulator type from the raw quadrant values and
 *                                                           rounded ONCE to the operand type
 *   orc_sw_gemm   src/cuda/strassen_reference_l1.cuh:12-117 level 1: 7 half-size products accumulated in the
 *                                                           accumulator type, postsums v1,v2,v3 in that type,
 *                                                           one rounding to the output type
 *                 include/cutlass/gemm/device/strassen_gemm.h:1764-1917
 *                                                           level 2: the same outer formulas with every outer
 *                                                           product computed by a level-1 recursion; the outer
 *                                                           hand-off buffers (M0, V1, V2, M4) are held in the
 *                                                           OUTPUT type when interim_round != 0 (the reference
 *                                                           kernels' behaviour) or in the accumulator type
 *                                                           when interim_round == 0
 *
 * The per-element sums are formed in exactly the reference order (k ascending, separate multiply and add,
 * no fused contraction: build with -ffp-contract=off), so on the same inputs this file and the reference
 * sources compiled for the host agree bit for bit; oracle/Makefile builds both and tests/ pins that.
 *
 * Parity pin: the reference stores no golden vectors for this path (its tests generate inputs at run
 * time and compare against its device oracle), so this restatement is pinned against the reference's
 * oracle sources compiled for the host (oracle/_ref) and against fixtures generated from that build.
 *
 * Type sets (dtype argument):
 *   0  f16 : A,B,C IEEE half; scalar and accumulator float   (harness instantiation <half,half,half,float,float>)
 *   1  f32 : everything float
 *   2  f64 : everything double (also the "truth" used for error measurement)
 *   3  tf32: float storage; every multiplicand is rounded to TF32 (10-bit mantissa, round-to-nearest-even
 *            on the dropped 13 bits) before the multiply; accumulate in float.  The reference has no
 *            oracle of this kind; it models the tensor-core input conversion and is used for tolerance
 *            tests only, never for bit-exact claims.
 *   4  bf16: A,B,C bfloat16 (round-to-nearest-even conversions); scalar and accumulator float.  The same
 *            generic bodies as the f16 set with the storage type exchanged, pinned against the reference's
 *            oracle templates instantiated for bfloat16 storage (the reference's harness itself has no
 *            bfloat16 case).
 *
 * Row sampling: every routine takes (nrows, rows).  rows == NULL means all rows of the (quadrant) row
 * space.  For orc_gemm a listed row r produces C row r.  For orc_sw_gemm at level 1 a listed row r in
 * [0, M/2) produces C rows r and r + M/2; at level 2 a listed row r in [0, M/4) produces C rows r,
 * r + M/4, r + M/2 and r + 3M/4.  Output is always written at its natural place in C (leading
 * dimension ldc); unlisted rows are not touched.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 half_t;
typedef __bf16 bf16_t;

static inline float tf32_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x; /* inf / nan */
  uint32_t lsb = (u >> 13) & 1u;
  u += 0xfffu + lsb;
  u &= 0xffffe000u;
  float y;
  memcpy(&y, &u, 4);
  return y;
}

/* ---------------------------------------------------------------------------------------------
 * Generic bodies, instantiated per type set by macro.
 *   TIN  operand storage type, TOUT output storage type, TACC accumulator/scalar type
 *   CVT(x) conversion applied to a multiplicand (identity except tf32)
 * ------------------------------------------------------------------------------------------- */

#define DEFINE_ORACLE(SUFFIX, TIN, TOUT, TACC, CVT)                                                     \
                                                                                                        \
  /* rows of C = alpha * A*B + beta * C ; A: MxK (lda), B: KxN (ldb) */                                 \
  static void gemm_rows_##SUFFIX(int M, int N, int K, TACC alpha, const TIN *A, int lda,                \
                                 const TIN *B, int ldb, TACC beta, const TOUT *Cin, TOUT *C, int ldc,   \
                                 int nrows, const int *rows) {                                          \
    int R = rows ? nrows : M;                                                                           \
    _Pragma("omp parallel") {                                                                           \
      TACC *acc = (TACC *)malloc(sizeof(TACC) * (size_t)N);                                             \
      _Pragma("omp for schedule(dynamic, 1)") for (int ri = 0; ri < R; ++ri) {                          \
        int i = rows ? rows[ri] : ri;                                                                   \
        for (int j = 0; j < N; ++j) acc[j] = (TACC)0;                                                   \
        for (int k = 0; k < K; ++k) {                                                                   \
          TACC a = CVT((TACC)A[(size_t)i * lda + k]);                                                   \
          const TIN *brow = B + (size_t)k * ldb;                                                        \
          for (int j = 0; j < N; ++j) acc[j] += a * CVT((TACC)brow[j]);                                 \
        }                                                                                               \
        for (int j = 0; j < N; ++j) {                                                                   \
          TACC c = (beta != (TACC)0) ? (TACC)Cin[(size_t)i * ldc + j] : (TACC)0;                        \
          TACC out = alpha * acc[j] + beta * c;                                                         \
          C[(size_t)i * ldc + j] = (TOUT)out;                                                           \
        }                                                                                               \
      }                                                                                                 \
      free(acc);                                                                                        \
    }                                                                                                   \
  }                                                                                                     \
                                                                                                        \
  /* The eight presums as packed quadrant matrices.                                                     \
   * pa: 4 matrices [hm x hk] in the order S1, S2, A02, A1S2                                            \
   * pb: 4 matrices [hk x hn] in the order B10, B31, S3, S3B2 */                                        \
  static void presums_##SUFFIX(int M, int N, int K, const TIN *A, int lda, const TIN *B, int ldb,       \
                               TIN *pa, TIN *pb) {                                                      \
    int hm = M / 2, hn = N / 2, hk = K / 2;                                                             \
    size_t qa = (size_t)hm * hk, qb = (size_t)hk * hn;                                                  \
    if (pa) {                                                                                           \
      _Pragma("omp parallel for") for (int r = 0; r < hm; ++r) for (int k = 0; k < hk; ++k) {           \
        TACC a0 = (TACC)A[(size_t)r * lda + k], a1 = (TACC)A[(size_t)r * lda + hk + k];                 \
        TACC a2 = (TACC)A[(size_t)(hm + r) * lda + k], a3 = (TACC)A[(size_t)(hm + r) * lda + hk + k];   \
        TACC s1 = a2 + a3;                                                                              \
        TACC s2 = s1 - a0;                                                                              \
        TACC a02 = a0 - a2;                                                                             \
        TACC a1s2 = a1 - s2;                                                                            \
        size_t o = (size_t)r * hk + k;                                                                  \
        pa[0 * qa + o] = (TIN)s1;                                                                       \
        pa[1 * qa + o] = (TIN)s2;                                                                       \
        pa[2 * qa + o] = (TIN)a02;                                                                      \
        pa[3 * qa + o] = (TIN)a1s2;                                                                     \
      }                                                                                                 \
    }                                                                                                   \
    if (pb) {                                                                                           \
      _Pragma("omp parallel for") for (int k = 0; k < hk; ++k) for (int c = 0; c < hn; ++c) {           \
        TACC b0 = (TACC)B[(size_t)k * ldb + c], b1 = (TACC)B[(size_t)k * ldb + hn + c];                 \
        TACC b2 = (TACC)B[(size_t)(hk + k) * ldb + c], b3 = (TACC)B[(size_t)(hk + k) * ldb + hn + c];   \
        TACC b10 = b1 - b0;                                                                             \
        TACC b31 = b3 - b1;                                                                             \
        TACC s3 = b31 + b0;                                                                             \
        TACC s3b2 = s3 - b2;                                                                            \
        size_t o = (size_t)k * hn + c;                                                                  \
        pb[0 * qb + o] = (TIN)b10;                                                                      \
        pb[1 * qb + o] = (TIN)b31;                                                                      \
        pb[2 * qb + o] = (TIN)s3;                                                                       \
        pb[3 * qb + o] = (TIN)s3b2;                                                                     \
      }                                                                                                 \
    }                                                                                                   \
  }                                                                                                     \
                                                                                                        \
  /* one accumulator row: acc[0..hn) = sum_k a[k] * Bm[k][0..hn) , k ascending */                       \
  static inline void prod_row_##SUFFIX(int hn, int hk, const TIN *a, const TIN *Bm, int ldbm,           \
                                       TACC *acc) {                                                     \
    for (int j = 0; j < hn; ++j) acc[j] = (TACC)0;                                                      \
    for (int k = 0; k < hk; ++k) {                                                                      \
      TACC av = CVT((TACC)a[k]);                                                                        \
      const TIN *brow = Bm + (size_t)k * ldbm;                                                          \
      for (int j = 0; j < hn; ++j) acc[j] += av * CVT((TACC)brow[j]);                                   \
    }                                                                                                   \
  }                                                                                                     \
                                                                                                        \
  /* Level-1 Strassen-Winograd on listed quadrant rows.  If accout != NULL the four quadrant            \
   * accumulators (before alpha/beta and output rounding) are ALSO written there as an M x N matrix     \
   * of TACC with leading dimension N (used by the level-2 recursion). */                              \
  static void sw1_rows_##SUFFIX(int M, int N, int K, TACC alpha, const TIN *A, int lda, const TIN *B,   \
                                int ldb, TACC beta, const TOUT *Cin, TOUT *C, int ldc, int nrows,       \
                                const int *rows, TACC *accout) {                                        \
    int hm = M / 2, hn = N / 2, hk = K / 2;                                                             \
    size_t qb = (size_t)hk * hn;                                                                        \
    TIN *pb = (TIN *)malloc(sizeof(TIN) * 4 * qb);                                                      \
    presums_##SUFFIX(M, N, K, A, lda, B, ldb, NULL, pb);                                                \
    const TIN *B0 = B, *B2 = B + (size_t)hk * ldb, *B3 = B + (size_t)hk * ldb + hn;                     \
    const TIN *B10 = pb, *B31 = pb + qb, *S3 = pb + 2 * qb, *S3B2 = pb + 3 * qb;                        \
    int R = rows ? nrows : hm;                                                                          \
    _Pragma("omp parallel") {                                                                           \
      TIN *pa = (TIN *)malloc(sizeof(TIN) * 4 * (size_t)hk);                                            \
      TACC *m = (TACC *)malloc(sizeof(TACC) * 7 * (size_t)hn);                                          \
      _Pragma("omp for schedule(dynamic, 1)") for (int ri = 0; ri < R; ++ri) {                          \
        int r = rows ? rows[ri] : ri;                                                                   \
        const TIN *a0 = A + (size_t)r * lda, *a1 = a0 + hk;                                             \
        const TIN *a2 = A + (size_t)(hm + r) * lda, *a3 = a2 + hk;                                      \
        TIN *s1 = pa, *s2 = pa + hk, *a02 = pa + 2 * hk, *a1s2 = pa + 3 * hk;                           \
        for (int k = 0; k < hk; ++k) {                                                                  \
          TACC x0 = (TACC)a0[k], x1 = (TACC)a1[k], x2 = (TACC)a2[k], x3 = (TACC)a3[k];                  \
          TACC t1 = x2 + x3;                                                                            \
          TACC t2 = t1 - x0;                                                                            \
          TACC t02 = x0 - x2;                                                                           \
          TACC t12 = x1 - t2;                                                                           \
          s1[k] = (TIN)t1;                                                                              \
          s2[k] = (TIN)t2;                                                                              \
          a02[k] = (TIN)t02;                                                                            \
          a1s2[k] = (TIN)t12;                                                                           \
        }                                                                                               \
        TACC *m0 = m, *m1 = m + hn, *m2 = m + 2 * hn, *m3 = m + 3 * hn, *m4 = m + 4 * hn,               \
             *m5 = m + 5 * hn, *m6 = m + 6 * hn;                                                        \
        prod_row_##SUFFIX(hn, hk, a0, B0, ldb, m0);                                                     \
        prod_row_##SUFFIX(hn, hk, a1, B2, ldb, m1);                                                     \
        prod_row_##SUFFIX(hn, hk, s2, S3, hn, m2);                                                      \
        prod_row_##SUFFIX(hn, hk, a02, B31, hn, m3);                                                    \
        prod_row_##SUFFIX(hn, hk, s1, B10, hn, m4);                                                     \
        prod_row_##SUFFIX(hn, hk, a1s2, B3, ldb, m5);                                                   \
        prod_row_##SUFFIX(hn, hk, a3, S3B2, hn, m6);                                                    \
        for (int j = 0; j < hn; ++j) {                                                                  \
          TACC v1 = m0[j] + m2[j];                                                                      \
          TACC v2 = v1 + m3[j];                                                                         \
          TACC v3 = v1 + m4[j];                                                                         \
          TACC q[4];                                                                                    \
          q[0] = m0[j] + m1[j];                                                                         \
          q[1] = v3 + m5[j];                                                                            \
          q[2] = v2 - m6[j];                                                                            \
          q[3] = v2 + m4[j];                                                                            \
          for (int h = 0; h < 4; ++h) {                                                                 \
            size_t i = (size_t)((h >> 1) ? hm + r : r), jj = (size_t)((h & 1) ? hn + j : j);            \
            if (accout) accout[i * (size_t)N + jj] = q[h];                                              \
            if (C) {                                                                                    \
              TACC c = (beta != (TACC)0) ? (TACC)Cin[i * ldc + jj] : (TACC)0;                           \
              TACC out = alpha * q[h] + beta * c;                                                       \
              C[i * ldc + jj] = (TOUT)out;                                                              \
            }                                                                                           \
          }                                                                                             \
        }                                                                                               \
      }                                                                                                 \
      free(pa);                                                                                         \
      free(m);                                                                                          \
    }                                                                                                   \
    free(pb);                                                                                           \
  }                                                                                                     \
                                                                                                        \
  /* Level 2: outer Winograd formulas, each outer product by a level-1 recursion.  With a row list      \
   * (rows q of the innermost quadrants, in [0, M/4)) only C rows q, q + M/4, q + M/2 and q + 3M/4 are  \
   * formed. */                                                                                         \
  static int sw2_##SUFFIX(int M, int N, int K, TACC alpha, const TIN *A, int lda, const TIN *B,         \
                          int ldb, TACC beta, const TOUT *Cin, TOUT *C, int ldc, int interim_round,     \
                          int nrows, const int *rows) {                                                 \
    int hm = M / 2, hn = N / 2, hk = K / 2;                                                             \
    size_t qa = (size_t)hm * hk, qb = (size_t)hk * hn, qc = (size_t)hm * hn;                            \
    TIN *pa = (TIN *)malloc(sizeof(TIN) * 4 * qa);                                                      \
    TIN *pb = (TIN *)malloc(sizeof(TIN) * 4 * qb);                                                      \
    TACC *mm = (TACC *)malloc(sizeof(TACC) * 7 * qc);                                                   \
    if (!pa || !pb || !mm) { free(pa); free(pb); free(mm); return 2; }                                  \
    presums_##SUFFIX(M, N, K, A, lda, B, ldb, pa, pb);                                                  \
    const TIN *opa[7] = {A, A + hk, pa + qa, pa + 2 * qa, pa, pa + 3 * qa, A + (size_t)hm * lda + hk};  \
    int olda[7] = {lda, lda, hk, hk, hk, hk, lda};                                                      \
    const TIN *opb[7] = {B, B + (size_t)hk * ldb, pb + 2 * qb, pb + qb, pb,                             \
                         B + (size_t)hk * ldb + hn, pb + 3 * qb};                                       \
    int oldb[7] = {ldb, ldb, hn, hn, hn, ldb, hn};                                                      \
    for (int p = 0; p < 7; ++p)                                                                         \
      sw1_rows_##SUFFIX(hm, hn, hk, (TACC)1, opa[p], olda[p], opb[p], oldb[p], (TACC)0, NULL, NULL, 0,  \
                        nrows, rows, mm + p * qc);                                                      \
    int R2 = rows ? 2 * nrows : hm;                                                                     \
    _Pragma("omp parallel for") for (int ri = 0; ri < R2; ++ri) for (int j = 0; j < hn; ++j) {          \
      int r = rows ? rows[ri >> 1] + ((ri & 1) ? hm / 2 : 0) : ri;                                      \
      size_t o = (size_t)r * hn + j;                                                                    \
      TACC m0 = mm[o], m1 = mm[qc + o], m2 = mm[2 * qc + o], m3 = mm[3 * qc + o];                       \
      TACC m4 = mm[4 * qc + o], m5 = mm[5 * qc + o], m6 = mm[6 * qc + o];                               \
      TACC q[4];                                                                                        \
      if (interim_round) {                                                                              \
        /* hand-off buffers held in the output type, hop by hop */                                      \
        TACC m0s = (TACC)(TOUT)m0;                                                                      \
        TACC v1s = (TACC)(TOUT)(m2 + m0s);                                                              \
        TACC v2s = (TACC)(TOUT)(m3 + v1s);                                                              \
        TACC m4s = (TACC)(TOUT)m4;                                                                      \
        q[0] = m1 + m0s;                                                                                \
        q[1] = m5 + v1s + m4s;                                                                          \
        q[2] = v2s - m6;                                                                                \
        q[3] = m4 + v2s;                                                                                \
      } else {                                                                                          \
        TACC v1 = m0 + m2;                                                                              \
        TACC v2 = v1 + m3;                                                                              \
        TACC v3 = v1 + m4;                                                                              \
        q[0] = m0 + m1;                                                                                 \
        q[1] = v3 + m5;                                                                                 \
        q[2] = v2 - m6;                                                                                 \
        q[3] = v2 + m4;                                                                                 \
      }                                                                                                 \
      for (int h = 0; h < 4; ++h) {                                                                     \
        size_t i = (size_t)((h >> 1) ? hm + r : r), jj = (size_t)((h & 1) ? hn + j : j);                \
        TACC c = (beta != (TACC)0) ? (TACC)Cin[i * ldc + jj] : (TACC)0;                                 \
        TACC out = alpha * q[h] + beta * c;                                                             \
        C[i * ldc + jj] = (TOUT)out;                                                                    \
      }                                                                                                 \
    }                                                                                                   \
    free(pa);                                                                                           \
    free(pb);                                                                                           \
    free(mm);                                                                                           \
    return 0;                                                                                           \
  }

#define IDENT(x) (x)
DEFINE_ORACLE(f16, half_t, half_t, float, IDENT)
DEFINE_ORACLE(f32, float, float, float, IDENT)
DEFINE_ORACLE(f64, double, double, double, IDENT)
DEFINE_ORACLE(tf32, float, float, float, tf32_round)
DEFINE_ORACLE(bf16, bf16_t, bf16_t, float, IDENT)

/* ------------------------------------------------------------------------------------------- */
/* C entry points (bound with ctypes by the tests).  Return 0 on success, 1 on bad arguments.   */

int orc_gemm(int dtype, int M, int N, int K, double alpha, const void *A, int lda, const void *B, int ldb,
             double beta, const void *Cin, void *C, int ldc, int nrows, const int *rows) {
  if (M <= 0 || N <= 0 || K <= 0 || !A || !B || !C) return 1;
  switch (dtype) {
    case 0: gemm_rows_f16(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, nrows, rows); return 0;
    case 1: gemm_rows_f32(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, nrows, rows); return 0;
    case 2: gemm_rows_f64(M, N, K, alpha, A, lda, B, ldb, beta, Cin, C, ldc, nrows, rows); return 0;
    case 3: gemm_rows_tf32(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, nrows, rows); return 0;
    case 4: gemm_rows_bf16(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, nrows, rows); return 0;
  }
  return 1;
}

/* level 0: naive; level 1: Strassen-Winograd (falls back to naive for odd sizes, exactly as the
 * reference's ReferenceStrassenWinogradGemm does, strassen_reference_l1.cuh:236-239); level 2: recursion. */
int orc_sw_gemm(int dtype, int level, int M, int N, int K, double alpha, const void *A, int lda, const void *B,
                int ldb, double beta, const void *Cin, void *C, int ldc, int nrows, const int *rows,
                int interim_round) {
  if (M <= 0 || N <= 0 || K <= 0 || !A || !B || !C) return 1;
  if (level == 0 || (level == 1 && ((M % 2) || (N % 2) || (K % 2))))
    return orc_gemm(dtype, M, N, K, alpha, A, lda, B, ldb, beta, Cin, C, ldc, nrows, rows);
  if (level == 1) {
    switch (dtype) {
      case 0: sw1_rows_f16(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, nrows, rows, NULL); return 0;
      case 1: sw1_rows_f32(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, nrows, rows, NULL); return 0;
      case 2: sw1_rows_f64(M, N, K, alpha, A, lda, B, ldb, beta, Cin, C, ldc, nrows, rows, NULL); return 0;
      case 3: sw1_rows_tf32(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, nrows, rows, NULL); return 0;
      case 4: sw1_rows_bf16(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, nrows, rows, NULL); return 0;
    }
    return 1;
  }
  if (level == 2) {
    if ((M % 4) || (N % 4) || (K % 4)) return 1;
    switch (dtype) {
      case 0: return sw2_f16(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, interim_round, nrows, rows);
      case 1: return sw2_f32(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, interim_round, nrows, rows);
      case 2: return sw2_f64(M, N, K, alpha, A, lda, B, ldb, beta, Cin, C, ldc, interim_round, nrows, rows);
      case 3: return sw2_tf32(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, interim_round, nrows, rows);
      case 4: return sw2_bf16(M, N, K, (float)alpha, A, lda, B, ldb, (float)beta, Cin, C, ldc, interim_round, nrows, rows);
    }
  }
  return 1;
}

/* pa: S1,S2,A02,A1S2 packed [4][M/2][K/2]; pb: B10,B31,S3,S3B2 packed [4][K/2][N/2]; operand type. */
int orc_sw_presums(int dtype, int M, int N, int K, const void *A, int lda, const void *B, int ldb, void *pa,
                   void *pb) {
  if ((M % 2) || (N % 2) || (K % 2) || !A || !B) return 1;
  switch (dtype) {
    case 0: presums_f16(M, N, K, A, lda, B, ldb, pa, pb); return 0;
    case 1:
    case 3: presums_f32(M, N, K, A, lda, B, ldb, pa, pb); return 0;
    case 2: presums_f64(M, N, K, A, lda, B, ldb, pa, pb); return 0;
    case 4: presums_bf16(M, N, K, A, lda, B, ldb, pa, pb); return 0;
  }
  return 1;
}

/* Truth for error measurement: rows of A*B in double from operands of any type set. */
int orc_truth_rows(int dtype, int M, int N, int K, const void *A, int lda, const void *B, int ldb, double *C,
                   int nrows, const int *rows) {
  if (!rows || nrows <= 0) return 1;
  (void)M;
#pragma omp parallel for schedule(dynamic, 1)
  for (int ri = 0; ri < nrows; ++ri) {
    int i = rows[ri];
    double *acc = C + (size_t)ri * N;
    for (int j = 0; j < N; ++j) acc[j] = 0.0;
    for (int k = 0; k < K; ++k) {
      double a;
      if (dtype == 0) a = (double)((const half_t *)A)[(size_t)i * lda + k];
      else if (dtype == 4) a = (double)(float)((const bf16_t *)A)[(size_t)i * lda + k];
      else if (dtype == 2) a = ((const double *)A)[(size_t)i * lda + k];
      else a = (double)((const float *)A)[(size_t)i * lda + k];
      if (dtype == 0) {
        const half_t *b = (const half_t *)B + (size_t)k * ldb;
        for (int j = 0; j < N; ++j) acc[j] += a * (double)b[j];
      } else if (dtype == 4) {
        const bf16_t *b = (const bf16_t *)B + (size_t)k * ldb;
        for (int j = 0; j < N; ++j) acc[j] += a * (double)(float)b[j];
      } else if (dtype == 2) {
        const double *b = (const double *)B + (size_t)k * ldb;
        for (int j = 0; j < N; ++j) acc[j] += a * b[j];
      } else {
        const float *b = (const float *)B + (size_t)k * ldb;
        for (int j = 0; j < N; ++j) acc[j] += a * (double)b[j];
      }
    }
  }
  return 0;
}
