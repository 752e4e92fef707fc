// Host-side operator: checks, workspace layout, tensor maps, launches.  See sw_host.h.
#include "sw_host.h"

#include <cuda.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "sw_kernel.cuh"
#include "sw_kernel_pair.cuh"
#include "sw_programs.h"

namespace sb200 {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major view -> tensor map with a [box_rows x 128 bytes] box and 128-byte swizzle.
int make_tmap(CUtensorMap* m, int esize, const View& v, int box_rows, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return kErrInternal;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(v.cols), static_cast<cuuint64_t>(v.rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(v.ld) * esize};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / esize), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(m, dt, 2, const_cast<void*>(v.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kErrInternal;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int esize_of(DType t) { return t == kF16 ? 2 : 4; }

struct Layout {
  int esize, bn, level;
  int mq, nq, kq;          // extents of one operand/output block (level 0: the whole matrix)
  int tiles_m, tiles_n, num_k;
  size_t off_status, off_pa, off_pb, off_ws[SB200_NUM_WS], total;
};

Layout make_layout(const GemmArgs& a) {
  Layout L;
  memset(&L, 0, sizeof(L));
  L.esize = esize_of(a.dtype);
  L.bn = a.bn == 128 ? 128 : 256;
  L.level = a.variant == kCubic ? 0 : 1;
  int div = L.level ? 2 : 1;
  L.mq = a.m / div;
  L.nq = a.n / div;
  L.kq = a.k / div;
  L.tiles_m = ceil_div(L.mq, a.pair ? 256 : 128);
  L.tiles_n = ceil_div(L.nq, L.bn);
  L.num_k = ceil_div(L.kq, 128 / L.esize);
  size_t off = 0;
  L.off_status = off;
  off += 256;
  if (a.variant == kInterleavedPresum) {
    L.off_pa = off;
    off = align_up(off + size_t(4) * L.mq * L.kq * L.esize, 256);
    L.off_pb = off;
    off = align_up(off + size_t(4) * L.kq * L.nq * L.esize, 256);
  }
  int nws = a.variant == kCubic ? 0 : (a.variant == kInterleavedPresum ? 4 : 2);
  size_t tile_bytes = size_t(128) * L.bn * sizeof(float);
  for (int i = 0; i < nws; ++i) {
    L.off_ws[i] = off;
    off = align_up(off + size_t(L.tiles_m) * L.tiles_n * (a.pair ? 2 : 1) * tile_bytes, 256);
  }
  L.total = off;
  return L;
}

template <typename Cfg>
int launch(const KernelParams& p, int grid, cudaStream_t stream) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(sw_tile_program_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  sw_tile_program_kernel<Cfg><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <int ESIZE, int BN>
int launch_mode(int mode, const KernelParams& p, int grid, cudaStream_t stream) {
  constexpr int STAGES = (BN == 256) ? 4 : 6;
  switch (mode) {
    case kPresumNone: return launch<KernelConfig<ESIZE, BN, STAGES, kPresumNone>>(p, grid, stream);
    case kPresumFeed: return launch<KernelConfig<ESIZE, BN, STAGES, kPresumFeed>>(p, grid, stream);
    case kPresumJob: return launch<KernelConfig<ESIZE, BN, STAGES, kPresumJob>>(p, grid, stream);
  }
  return kErrInternal;
}

int launch_any(int esize, int bn, int mode, const KernelParams& p, int grid, cudaStream_t stream);
int launch_any_pair(int esize, int mode, const KernelParams& p, int pairs, cudaStream_t stream);

int launch_any(int esize, int bn, int mode, const KernelParams& p, int grid, cudaStream_t stream) {
  if (bn < 0) return launch_any_pair(esize, mode, p, grid, stream);
  if (esize == 2 && bn == 256) return launch_mode<2, 256>(mode, p, grid, stream);
  if (esize == 2 && bn == 128) return launch_mode<2, 128>(mode, p, grid, stream);
  if (esize == 4 && bn == 256) return launch_mode<4, 256>(mode, p, grid, stream);
  if (esize == 4 && bn == 128) return launch_mode<4, 128>(mode, p, grid, stream);
  return kErrNotSupported;
}

template <typename Cfg>
int launch_pair(const KernelParams& p, int pairs, cudaStream_t stream) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(sw_tile_program_pair_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, sw_tile_program_pair_kernel<Cfg>, p));
}

template <int ESIZE>
int launch_pair_mode(int mode, const KernelParams& p, int pairs, cudaStream_t stream) {
  constexpr int STAGES = 6;
  if (mode == kPresumNone && getenv("SB200_STAGES7")) return launch_pair<PairConfig<ESIZE, 7, kPresumNone>>(p, pairs, stream);
  switch (mode) {
    case kPresumNone: return launch_pair<PairConfig<ESIZE, STAGES, kPresumNone>>(p, pairs, stream);
    case kPresumFeed: return launch_pair<PairConfig<ESIZE, STAGES, kPresumFeed>>(p, pairs, stream);
    case kPresumJob: return launch_pair<PairConfig<ESIZE, STAGES, kPresumJob>>(p, pairs, stream);
  }
  return kErrInternal;
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

int launch_any_pair(int esize, int mode, const KernelParams& p, int pairs, cudaStream_t stream) {
  if (esize == 2) return launch_pair_mode<2>(mode, p, pairs, stream);
  if (esize == 4) return launch_pair_mode<4>(mode, p, pairs, stream);
  return kErrNotSupported;
}

}  // namespace

int can_implement(const GemmArgs& a) {
  if (a.m <= 0 || a.n <= 0 || a.k <= 0 || !a.a || !a.b || !a.d) return kErrInvalidProblem;
  if (a.dtype != kF16 && a.dtype != kF32) return kErrNotSupported;
  if (a.bn != 0 && a.bn != 128 && a.bn != 256) return kErrNotSupported;
  if (a.pair && a.bn == 128) return kErrNotSupported;
  const int es = esize_of(a.dtype);
  const int vec = 16 / es;  // elements per 16 bytes
  const int div = a.variant == kCubic ? 1 : 2;
  if (div == 2 && ((a.m % 2) || (a.n % 2) || (a.k % 2))) return kErrInvalidProblem;
  // every quadrant row must start on a 16-byte boundary (TMA base/stride rule, vector loads and stores)
  if ((a.k / div) % vec || (a.n / div) % vec) return kErrMisalignedOperand;
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) | reinterpret_cast<uintptr_t>(a.d)) & 15)
    return kErrMisalignedOperand;
  return kOk;
}

size_t workspace_bytes(const GemmArgs& a) { return make_layout(a).total; }

WorkspaceLayout workspace_layout(const GemmArgs& a) {
  const Layout L = make_layout(a);
  WorkspaceLayout w;
  memset(&w, 0, sizeof(w));
  w.status = L.off_status;
  w.presum_a = L.off_pa;
  w.presum_b = L.off_pb;
  for (int i = 0; i < SB200_NUM_WS; ++i) w.handoff[i] = L.off_ws[i];
  w.total = L.total;
  w.mq = L.mq; w.nq = L.nq; w.kq = L.kq;
  w.tiles_m = L.tiles_m; w.tiles_n = L.tiles_n; w.bn = L.bn;
  return w;
}

int launches_per_run(const GemmArgs& a) { return a.variant == kInterleavedPresum ? 2 : 1; }

int run(const GemmArgs& a, void* workspace, size_t workspace_size, cudaStream_t stream) {
  int rc = can_implement(a);
  if (rc) return rc;
  const Layout L = make_layout(a);
  if (!workspace) return kErrWorkspaceNull;
  if (workspace_size < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255)) return kErrWorkspaceNull;
  char* wsb = static_cast<char*>(workspace);
  const int es = L.esize;

  KernelParams p;
  memset(&p, 0, sizeof(p));
  p.status = reinterpret_cast<int*>(wsb + L.off_status);
  cudaError_t ce = cudaMemsetAsync(p.status, 0, 256, stream);
  if (ce != cudaSuccess) return static_cast<int>(ce);

  const char* A = static_cast<const char*>(a.a);
  const char* B = static_cast<const char*>(a.b);
  char* D = static_cast<char*>(a.d);
  const long long lda = a.k, ldb = a.n, ldd = a.n;
  if (L.level == 0) {
    for (int v = 0; v < 8; ++v) p.view[v] = View{A, lda, a.m, a.k};
    for (int v = 8; v < 16; ++v) p.view[v] = View{B, ldb, a.k, a.n};
    p.out[0] = D;
  } else {
    for (int q = 0; q < 4; ++q) {
      p.view[SB200_VIEW_A0 + q] = View{A + ((q >> 1) * L.mq * lda + (q & 1) * L.kq) * es, lda, L.mq, L.kq};
      p.view[SB200_VIEW_B0 + q] = View{B + ((q >> 1) * L.kq * ldb + (q & 1) * L.nq) * es, ldb, L.kq, L.nq};
      p.out[q] = D + ((q >> 1) * L.mq * ldd + (q & 1) * L.nq) * es;
      if (a.variant == kInterleavedPresum) {
        p.view[SB200_VIEW_PA0 + q] =
            View{wsb + L.off_pa + size_t(q) * L.mq * L.kq * es, static_cast<long long>(L.kq), L.mq, L.kq};
        p.view[SB200_VIEW_PB0 + q] =
            View{wsb + L.off_pb + size_t(q) * L.kq * L.nq * es, static_cast<long long>(L.nq), L.kq, L.nq};
      } else {
        p.view[SB200_VIEW_PA0 + q] = p.view[SB200_VIEW_A0 + q];
        p.view[SB200_VIEW_PB0 + q] = p.view[SB200_VIEW_B0 + q];
      }
    }
  }
  for (int v = 0; v < 8; ++v)
    if ((rc = make_tmap(&p.tmap[v], es, p.view[v], 128, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  // B tiles of 32-bit elements are deposited with 32-byte swizzle atoms (see KernelConfig::B_SWZ32)
  const CUtensorMapSwizzle b_swz = es == 4 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  for (int v = 8; v < 16; ++v)
    if ((rc = make_tmap(&p.tmap[v], es, p.view[v], 128 / es, b_swz))) return rc;
  p.ldo = ldd;
  p.out_rows = L.mq;
  p.out_cols = L.nq;
  for (int i = 0; i < SB200_NUM_WS; ++i) p.ws[i] = reinterpret_cast<float*>(wsb + L.off_ws[i]);
  p.tiles_m = L.tiles_m;
  p.tiles_n = L.tiles_n;
  p.num_k = L.num_k;
  p.band = 8;
  if (getenv("SB200_PROF")) {
    // measurement aid: per-CTA cycle counters of the CTA-pair kernels, printed by the next call
    static long long* prof_dev = nullptr;
    static long long prof_host[8 * 256];
    if (!prof_dev) {
      cudaMalloc(&prof_dev, sizeof(prof_host));
    } else {
      cudaDeviceSynchronize();
      cudaMemcpy(prof_host, prof_dev, sizeof(prof_host), cudaMemcpyDeviceToHost);
      double sum[8] = {0};
      int n = 0;
      for (int c = 0; c < 148; c += 2, ++n)
        for (int i = 0; i < 8; ++i) sum[i] += double(prof_host[c * 8 + i]);
      double psum3 = 0, psum4 = 0, e5 = 0, e6 = 0;
      for (int c = 1; c < 148; c += 2) { psum3 += double(prof_host[c * 8 + 3]); psum4 += double(prof_host[c * 8 + 4]); e5 += double(prof_host[c * 8 + 5]); e6 += double(prof_host[c * 8 + 6]); }
      fprintf(stderr, "[prof] leader mma thread: total %.0f = wait_full %.0f + wait_free %.0f + issue %.0f + commit %.0f + rest | producer A: wait_empty %.0f issue %.0f total %.0f\n",
              sum[0] / n, sum[1] / n, sum[2] / n, sum[5] / n, sum[6] / n, sum[3] / n, sum[7] / n, sum[4] / n);
      (void)psum3; (void)psum4; (void)e5; (void)e6;
    }
    cudaMemset(prof_dev, 0, sizeof(prof_host));
    p.prof = prof_dev;
  }
  if (const char* pf = getenv("SB200_PREFETCH")) p.prefetch_dist = atoi(pf);
  if (const char* bd = getenv("SB200_BAND")) p.band = atoi(bd) > 0 ? atoi(bd) : 8;
  if (const char* dbg = getenv("SB200_DEBUG_FLAGS")) p.debug_flags = atoi(dbg);
  p.job_pa = wsb + L.off_pa;
  p.job_pb = wsb + L.off_pb;
  p.job_mq = L.mq;
  p.job_nq = L.nq;
  p.job_kq = L.kq;

  int grid = L.tiles_m * L.tiles_n;
  int cap = a.sm_limit > 0 ? a.sm_limit : sm_count();
  if (a.pair) cap /= 2;  // one pair per two SMs
  if (grid > cap) grid = cap;
  const int bn_sel = a.pair ? -1 : L.bn;  // -1 routes launch_any to the CTA-pair kernels (grid = pairs)

  int nev = 0;
  auto mark = [&]() -> int {
    if (!a.events) return 0;
    return static_cast<int>(cudaEventRecord(a.events[nev++], stream));
  };
  if ((rc = mark())) return rc;
  switch (a.variant) {
    case kCubic:
      p.prog = programs::level0();
      rc = launch_any(es, bn_sel, kPresumNone, p, grid, stream);
      break;
    case kFusedPresum:
      p.prog = programs::level1_full(true);
      rc = launch_any(es, bn_sel, kPresumFeed, p, grid, stream);
      break;
    case kInterleavedPresum:
      p.prog = programs::level1_first();
      rc = launch_any(es, bn_sel, kPresumJob, p, grid, stream);
      if (rc) return rc;
      if ((rc = mark())) return rc;
      p.prog = getenv("SB200_L1_PLAIN") ? programs::level1_second() : programs::level1_second_taps();
      rc = launch_any(es, bn_sel, kPresumNone, p, grid, stream);
      break;
    default:
      return kErrNotSupported;
  }
  if (rc) return rc;
  return mark();
}

int read_status(void* workspace, cudaStream_t stream) {
  int st = 0;
  cudaError_t e = cudaMemcpyAsync(&st, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  return st;
}

}  // namespace sb200
