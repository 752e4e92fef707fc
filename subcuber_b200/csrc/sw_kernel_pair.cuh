// CTA-pair variant of the tile-program kernel: two CTAs of a 2-CTA cluster (two SMs) compute one 256 x 256 output
// tile with `tcgen05.mma.cta_group::2`.  Each CTA keeps its own 128 rows of A and its own 128 columns of B in
// shared memory and its own 128 rows of every accumulator in tensor memory; the tensor cores of both SMs read
// both halves of B.  Per MMA step a CTA therefore loads 32 KiB instead of 48 KiB (B traffic per SM halves), which
// is the sm_100 replacement for cluster-multicast loads and needs none: every TMA load here is a plain tiled load
// into the issuing CTA's own shared memory.
//
// Roles are those of sw_kernel.cuh, with these pair rules:
//   * both CTAs run a TMA producer for their own halves; the bytes of both are reported to the LEADER's (cluster
//     rank 0) full barrier, which the leader's producer arms with the pair's total;
//   * only the leader issues MMAs; its commits arrive on the stage-empty and slot-full barriers of BOTH CTAs;
//   * both CTAs run epilogue warps on their own TMEM half and return slot credits to the leader's slot-free barrier;
//   * in FEED mode the presum warps of both CTAs write their own shared memory and arrive on the leader's barrier.
#pragma once
#include "sw_kernel.cuh"

// Cycle counters for tuning are compiled in only on request; otherwise they cost nothing.
//   -DSB200_PROFILE           per-launch totals and the MMA issuer's waits for a free TMEM slot (two clock reads per product)
//   -DSB200_PROFILE_KSTEP     + clock reads around every k-step (MMA issuer, producer)
//   -DSB200_PROFILE_EPILOGUE  + epilogue step and segment timers
//   -DSB200_PROFILE_TRACE     + a per-k-step timeline of one tile (adds an observer warp)
#if defined(SB200_PROFILE_KSTEP) || defined(SB200_PROFILE_EPILOGUE) || defined(SB200_PROFILE_TRACE)
#ifndef SB200_PROFILE
#define SB200_PROFILE
#endif
#endif
#ifdef SB200_PROFILE
#define SB200_CLOCK_LIGHT() clock64()
#else
#define SB200_CLOCK_LIGHT() 0ll
#endif
#if defined(SB200_PROFILE_KSTEP) || defined(SB200_PROFILE_TRACE)
#define SB200_CLOCK() clock64()
#else
#define SB200_CLOCK() 0ll
#endif

namespace sb200 {

template <int ESIZE_, int STAGES_, int MODE_, bool SCALED_ = false>
struct PairConfig {
  static constexpr bool SCALED = SCALED_;  // D = alpha * sum + beta * C instead of D = sum
  static constexpr int ESIZE = ESIZE_;
  static constexpr int BM = 128;                  // rows per CTA
  static constexpr int PAIR_M = 256;              // rows per pair tile
  static constexpr int BN = 256;                  // columns per pair tile = accumulator columns per CTA
  static constexpr int BN_CTA = 128;              // columns of B held by each CTA
  static constexpr int BK = 128 / ESIZE;
  static constexpr int STAGES = STAGES_;
  static constexpr int MODE = MODE_;
  // fp32 sources an epilogue step may sum (hand-off tiles of the program, + one of the level above, + the partial
  // sum of a split tile).  The kernels with presum warps have a smaller register budget and run programs that
  // need fewer: JOB = first launch of the interleaved plan (1 + 1), FEED = one fused launch, never linked or split.
  static constexpr int NSRC_MAX = MODE_ == 0 ? SB200_MAX_SRC_TERMS + 1 : (MODE_ == 2 ? 2 : 1);
  // TMEM slots a step may sum: the programs of the kernels without presum warps read one slot per step
  static constexpr int NSLOT_MAX = MODE_ == 0 ? 1 : 2;
  static constexpr int UMMA_K = 32 / ESIZE;
  static constexpr int KSUB = BK / UMMA_K;
  static constexpr int A_BYTES = BM * 128;
  static constexpr int NBLK = BN_CTA * ESIZE / 128;
  static constexpr int BLK_BYTES = BK * 128;
  static constexpr int B_BYTES = NBLK * BLK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SLOTS = 2;
  static constexpr int TMEM_COLS = 512;
  static constexpr int PRESUM_WARPS = (MODE == kPresumNone) ? 0 : 4;
  // warps 0-5 as in sw_kernel.cuh; warps 6 and 7 = more TMA producers (see the producer section); presum warps follow
#ifdef SB200_PROFILE_TRACE
  static constexpr int FIRST_PRESUM_WARP = (MODE_ == kPresumNone) ? 9 : 8;  // warp 8 = full-barrier monitor (tracing)
#else
  static constexpr int FIRST_PRESUM_WARP = 8;
#endif
  static constexpr int THREADS = (FIRST_PRESUM_WARP + PRESUM_WARPS) * 32;
  static constexpr int BAR_BYTES = 1024;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + kStagingBytes + 1024;
  static constexpr uint32_t FMT = (ESIZE == 2) ? 0u : 2u;
  static constexpr bool B_SWZ32 = (ESIZE == 4);
  static constexpr uint32_t B_LAYOUT_TYPE = B_SWZ32 ? 1u : 2u;
  static constexpr uint32_t B_SBO = B_SWZ32 ? 512u : 1024u;
};

// How the roles of a CTA pair learn which unit comes next.
//   static   unit = pair + i * pairs: round-robin, wave after wave;
//   dynamic  the first producer warp of the leader CTA (the scheduler) draws the next unit number from a counter in
//            global memory when it needs one and publishes it to both CTAs through a small ring in shared memory;
//            every other role of both CTAs reads the ring in order.  Units are then started in raster order by
//            whichever pair is free: a pair on a faster part of the chip simply takes more tiles, and - what matters
//            more - tiles that are neighbours in raster order start close together in time, so the pairs that share
//            operand panels stay close in K and find them in L2.  (With the static deal the pairs drift apart by up to
//            a whole tile's time within a dozen tiles - measured on B200: their speeds differ by up to 6 % with their
//            position on the chip - and DRAM traffic doubles.)
// Ring protocol: sched_full[s] (one arrival: the scheduler, after it wrote the unit number into both CTAs' slot s) and
// the leader's sched_empty[s] (one arrival per consumer warp of the pair when it is done with the unit of slot s).
constexpr int kSchedSlots = 4;

struct UnitCursor {
  uint64_t* full;        // this CTA's sched_full[kSchedSlots]
  uint64_t* empty;       // sched_empty[kSchedSlots] (the leader's copy is the one that counts)
  int* slots;            // this CTA's unit numbers
  int* counter;          // global unit counter of this launch (dynamic), or null (static)
  volatile int* abort_flag;
  unsigned long long wait_ns;
  int pair, num_pairs, num_units;
  uint32_t i;            // units taken so far
  bool scheduler;        // this warp draws the units

  __device__ __forceinline__ void init(uint64_t* full_, uint64_t* empty_, int* slots_, const KernelParams& p, int pair_,
                                       int num_pairs_, bool scheduler_, volatile int* abort_flag_) {
    full = full_; empty = empty_; slots = slots_; counter = p.unit_counter; abort_flag = abort_flag_;
    wait_ns = p.wait_ns; pair = pair_; num_pairs = num_pairs_; num_units = total_units(p); i = 0;
    scheduler = scheduler_;
  }
  // Next unit number of this pair, the same in every lane; -1: no more units (or a wait was given up: *ok = false).
  __device__ __forceinline__ int next(bool* ok) {
    if (!counter) {
      const int u = pair + static_cast<int>(i) * num_pairs;
      return u < num_units ? u : -1;
    }
    const uint32_t s = i % kSchedSlots, round = i / kSchedSlots;
    int u = 0;
    if (scheduler) {
      bool got = true;
      if (round > 0) got = ptx::mbar_wait_warp<true>(&empty[s], (round - 1) & 1u, abort_flag, wait_ns);
      if (!got) { *ok = false; return -1; }
      if (ptx::elect_one()) {
        u = atomicAdd(counter, 1);
        slots[s] = u;
        ptx::st_shared_cluster_u32(&slots[s], 1, static_cast<uint32_t>(u));
        ptx::mbar_arrive_cluster(&full[s], 1);
        ptx::mbar_arrive_cluster(&full[s], 0);
      }
      __syncwarp();
    }
    if (!ptx::mbar_wait_warp<true>(&full[s], round & 1u, abort_flag, wait_ns)) { *ok = false; return -1; }
    u = slots[s];
    return u < num_units ? u : -1;
  }
  // This warp is done with the unit it took last.
  __device__ __forceinline__ void done(int lane) {
    if (counter) {
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(&empty[i % kSchedSlots], 0);
    }
    ++i;
  }
};

template <typename Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1) sw_tile_program_pair_kernel(const __grid_constant__ KernelParams p) {
  constexpr int ESIZE = Cfg::ESIZE;
  constexpr int BN = Cfg::BN;
  constexpr int BK = Cfg::BK;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int SLOTS = Cfg::SLOTS;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_base = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* slot_full = empty_bar + STAGES;
  uint64_t* slot_free = slot_full + SLOTS;
  uint64_t* sched_full = slot_free + SLOTS;
  uint64_t* sched_empty = sched_full + kSchedSlots;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(sched_empty + kSchedSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* sched_slots = reinterpret_cast<int*>(tmem_holder + 2);
  volatile int* presum_slot = sched_slots + kSchedSlots;   // chunk number handed around the presum warps
  const uint32_t staging = ptx::smem_u32(bar_base + Cfg::BAR_BYTES);  // epilogue staging rows (epilogue.cuh)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();   // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int nproducts = p.prog.nproducts;
  // warps of the pair that read the unit ring: 3 producers and 4 epilogue warps per CTA, the leader's MMA warp, and
  // the presum warps when they feed the stage ring
  constexpr int kRingReaders = 2 * (3 + 4 + (Cfg::MODE == kPresumFeed ? Cfg::PRESUM_WARPS : 0)) + 1;
  UnitCursor cursor;
  cursor.init(sched_full, sched_empty, sched_slots, p, pair, num_pairs, rank == 0 && warp == 0, abort_flag);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      // leader's full barrier: its own producer + (FEED) the presum warps of both CTAs
      ptx::mbar_init(&full_bar[s], 1 + (Cfg::MODE == kPresumFeed ? 2 * Cfg::PRESUM_WARPS : 0));
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < SLOTS; ++s) {
      ptx::mbar_init(&slot_full[s], 1);
      ptx::mbar_init(&slot_free[s], 8);  // 4 epilogue warps of each CTA
    }
    for (int s = 0; s < kSchedSlots; ++s) {
      ptx::mbar_init(&sched_full[s], 1);
      ptx::mbar_init(&sched_empty[s], kRingReaders);
    }
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_holder, Cfg::TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across the pair
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0 || warp == 6 || warp == 7) {
    // ------------------------------------------------------------------ TMA producers (both CTAs)
    // Measured on B200: the tiled loads of ONE warp complete one after the other, about 240 ns apiece whatever the
    // box holds (4 to 32 KiB), while loads of different warps overlap.  A k-step lasts about 370 ns, so a single
    // producer issuing two or three loads per k-step cannot keep up.  Three single-thread producers (warps 0, 6, 7)
    // take the k-steps in turn; each issues the A load and the B load of its k-step (B is one 3-D load when the B
    // maps are blocked) and, in the leader CTA, arms the full barrier with the pair's bytes.
    // Each producer warp runs its loop warp-uniformly and one elected lane issues (see ptx::elect_one).
    {
      const uint32_t my_turn = (warp == 0) ? 0u : static_cast<uint32_t>(warp - 5);
      uint32_t turn = 0;
      if (warp == 0 && lane == 0)
        for (int v = 0; v < SB200_NUM_VIEWS; ++v) ptx::prefetch_tmap(&p.tmap[v]);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const long long pt0 = SB200_CLOCK();
      long long pw_empty = 0, pw_issue = 0;
      for (int it = 0; ok; ++it, cursor.done(lane)) {
        const int unit = cursor.next(&ok);
        if (unit < 0) break;
        const WorkUnit wu = unit_of(p, unit);
        const TileCoord tile = tile_of(wu.tile, p.tiles_m, p.tiles_n, p.band);
        const int row0 = tile.i * Cfg::PAIR_M + static_cast<int>(rank) * Cfg::BM;
        // a column half of a tile: each CTA brings 64 of the half's 128 columns (half the column blocks of a B tile)
        const int col0 = tile.j * BN + wu.col_part * (BN / 2) + static_cast<int>(rank) * (Cfg::BN_CTA / wu.col_parts);
        bool panels_seen = !(Cfg::MODE == kPresumJob && p.panels.enabled);
        for (int ps = 0; ok && ps < nproducts; ++ps) {
          const sb200_product_t& pr = p.prog.product[ps];
          const bool a_tma = pr.a.nterms == 1;
          const bool b_tma = pr.b.nterms == 1;
          const int nblk = Cfg::NBLK / wu.col_parts;  // column blocks of B this CTA loads per k-step
          const uint32_t tx = 2u * ((a_tma ? Cfg::A_BYTES : 0) + (b_tma ? nblk * Cfg::BLK_BYTES : 0));  // both CTAs' bytes
          if (!panels_seen && ((pr.a.view[0] >= SB200_VIEW_PA0 && pr.a.view[0] < SB200_VIEW_B0) ||
                               pr.b.view[0] >= SB200_VIEW_PB0)) {
            // one-launch plan: the first product of a tile that reads presums waits (bounded) until the presum
            // warps of the grid have published the tile's A panel and B panel; TMA reads them through the async proxy.
            // It waits first for the LAST B panel of the group of tile columns that are in flight together: B panels
            // are published in column order, so without this the tiles of one wave would resume a few microseconds
            // apart per column and stay apart in K for the rest of the launch (tiles that share an operand panel find
            // it in L2 only while they read the same K range at the same time).
            int last_j = tile.j;
            if (p.panels.group_cols > 0) {
              last_j = (tile.j / p.panels.group_cols + 1) * p.panels.group_cols - 1;
              if (last_j >= p.tiles_n) last_j = p.tiles_n - 1;
            }
            const bool got = wait_counter(p.panels.ready_b + last_j, p.panels.chunks, abort_flag, p.wait_ns) &&
                             wait_counter(p.panels.ready_a + tile.i, p.panels.chunks, abort_flag, p.wait_ns) &&
                             wait_counter(p.panels.ready_b + tile.j, p.panels.chunks, abort_flag, p.wait_ns);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusPresumTimeout);
              ok = false;
              break;
            }
            ptx::fence_proxy_async_all();
            panels_seen = true;
          }
          const CUtensorMap* ma = &p.tmap[pr.a.view[0]];
          const CUtensorMap* mb = (wu.col_parts == 2 && p.b_blocked) ? &p.tmap_half_b[pr.b.view[0] - SB200_VIEW_B0]
                                                                     : &p.tmap[pr.b.view[0]];
          const bool no_load_all = SB200_DEBUG_BIT(p, 2);
          for (int kk = wu.k0; kk < wu.k1; ++kk) {
            const bool mine = (turn == my_turn);
            if (++turn == 3u) turn = 0;
            if (!mine) {
              if (++stage == STAGES) { stage = 0; phase ^= 1u; }
              continue;
            }
            const long long tw = SB200_CLOCK();
            // the stage-empty barrier is signalled by tcgen05.commit only: no cluster-scope acquire needed
            const bool got = ptx::mbar_wait_warp<false>(&empty_bar[stage], phase ^ 1u, abort_flag, p.wait_ns);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusProducerTimeout);
              ok = false;
              break;
            }
            const long long tw2 = SB200_CLOCK();
            pw_empty += tw2 - tw;
#ifdef SB200_PROFILE_TRACE
            const bool traced = p.prof && lane == 0 && blockIdx.x == 0 && it == 3 && ps == 0 && kk < 64;
            if (traced) p.prof[2048 + kk * 8 + 0] = tw2;
#endif
            uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
            uint8_t* sb = sa + Cfg::A_BYTES;
            // measurement aids: bit 1 = never load; bit 3 = load only while the ring fills for the first time
            const bool no_load = no_load_all || (SB200_DEBUG_BIT(p, 8) && (it != 0 || ps > 0 || kk >= wu.k0 + STAGES));
            if (ptx::elect_one()) {
              if (rank == 0) {
                if (tx && !no_load) ptx::mbar_arrive_expect_tx(&full_bar[stage], tx);
                else ptx::mbar_arrive(&full_bar[stage]);
              }
#ifdef SB200_PROFILE
              if (p.hint_mode && p.b_blocked && !no_load) {
                auto policy_of = [](int code) {
                  return code == 1 ? ptx::l2_policy_evict_first()
                                   : (code == 2 ? ptx::l2_policy_evict_last() : ptx::l2_policy_evict_normal());
                };
                const int ha = p.hint_mode / 10, hb = p.hint_mode % 10;
                if (a_tma) {
                  if (ha) ptx::tma_load_2d_pair_hint(sa, ma, &full_bar[stage], kk * BK, row0, policy_of(ha));
                  else ptx::tma_load_2d_pair(sa, ma, &full_bar[stage], kk * BK, row0);
                }
                if (b_tma) {
                  if (hb) ptx::tma_load_3d_pair_hint(sb, mb, &full_bar[stage], 0, kk * BK, col0 / BK, policy_of(hb));
                  else ptx::tma_load_3d_pair(sb, mb, &full_bar[stage], 0, kk * BK, col0 / BK);
                }
              } else
#endif
              {
              if (a_tma && !no_load) ptx::tma_load_2d_pair(sa, ma, &full_bar[stage], kk * BK, row0);
              if (b_tma && !no_load) {
                if (p.b_blocked) {
                  ptx::tma_load_3d_pair(sb, mb, &full_bar[stage], 0, kk * BK, col0 / BK);
                } else {
#pragma unroll
                  for (int nb = 0; nb < Cfg::NBLK; ++nb)
                    if (nb < nblk)
                      ptx::tma_load_2d_pair(sb + nb * Cfg::BLK_BYTES, mb, &full_bar[stage], col0 + nb * BK, kk * BK);
                }
              }
              }
            }
            __syncwarp();
            pw_issue += SB200_CLOCK() - tw2;
#ifdef SB200_PROFILE_TRACE
            if (traced) p.prof[2048 + kk * 8 + 1] = SB200_CLOCK();
#endif
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
#ifdef SB200_PROFILE
      if (p.prof && warp == 0 && lane == 0) {
        p.prof[blockIdx.x * 8 + 7] = pw_issue;
        p.prof[blockIdx.x * 8 + 3] = pw_empty;
        p.prof[blockIdx.x * 8 + 4] = SB200_CLOCK() - pt0;
      }
#else
      (void)pw_issue; (void)pw_empty; (void)pt0;
#endif
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    // The whole warp runs the loop (see ptx::elect_one); one elected lane issues the MMAs and the commits.
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t free_bits = 0;
      uint32_t iter = 0;
      bool ok = true;
      const long long mt0 = SB200_CLOCK_LIGHT();
      long long mw_full = 0, mw_free = 0, mw_issue = 0;
      for (int it = 0; ok; ++it, ++iter, cursor.done(lane)) {
        const int unit = cursor.next(&ok);
        if (unit < 0) break;
        const WorkUnit wu = unit_of(p, unit);
        const int nk = wu.k1 - wu.k0;
        const uint32_t sx = p.prog.alternate_slots ? (iter & 1u) : 0u;
#ifdef SB200_PROFILE
        // wall-clock time at which this pair starts its iter-th tile (skew between the pairs of a wave)
        if (p.prof && lane == 0 && iter < 128) {
          p.prof[4096 + pair * 128 + iter] = static_cast<long long>(ptx::globaltimer_ns());
          if (iter == 0) {
            unsigned smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            p.prof[3000 + pair] = smid;
          }
        }
#endif
        for (int ps = 0; ok && ps < nproducts; ++ps) {
          const sb200_product_t& pr = p.prog.product[ps];
          const uint32_t slot = pr.slot ^ sx;
          if (pr.wait_free) {
            const long long tw = SB200_CLOCK_LIGHT();
            const bool got = ptx::mbar_wait_warp<true>(&slot_free[slot], ((free_bits >> slot) & 1u) ^ 1u, abort_flag, p.wait_ns);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusMmaTimeout);
              ok = false;
              break;
            }
            mw_free += SB200_CLOCK_LIGHT() - tw;
            free_bits ^= (1u << slot);
            ptx::tc_fence_after_sync();
          }
          const uint32_t idesc = ptx::umma_idesc((ESIZE == 2 && p.bf16) ? 1u : Cfg::FMT, Cfg::PAIR_M, BN / wu.col_parts, pr.negate != 0);
          const uint32_t tmem_d = tmem_base + slot * BN;
          const bool skip_mma = SB200_DEBUG_BIT(p, 1);
          // descriptors differ between stages and k-substeps only in the start-address field (low word, 16-byte units)
          const uint64_t adesc0 = ptx::umma_desc_sw128(ptx::smem_u32(smem), 16, 1024);
          const uint64_t bdesc0 =
              ptx::umma_desc_sw128(ptx::smem_u32(smem) + Cfg::A_BYTES, Cfg::BLK_BYTES, Cfg::B_SBO, Cfg::B_LAYOUT_TYPE);
          for (int kk = 0; ok && kk < nk; ++kk) {
            const long long tw = SB200_CLOCK();
            // in FEED mode the peer's presum warps arrive on this barrier after writing their own shared memory
            // through the generic proxy: that hand-over needs the cluster-scope acquire; TMA-only stages do not
            const bool got = (Cfg::MODE == kPresumFeed)
                                 ? ptx::mbar_wait_warp<true>(&full_bar[stage], phase, abort_flag, p.wait_ns)
                                 : ptx::mbar_wait_warp<false>(&full_bar[stage], phase, abort_flag, p.wait_ns);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusMmaTimeout);
              ok = false;
              break;
            }
            const long long ti0 = SB200_CLOCK();
            mw_full += ti0 - tw;
            const uint64_t adesc_s = adesc0 + static_cast<uint64_t>((stage * Cfg::STAGE_BYTES) >> 4);
            const uint64_t bdesc_s = bdesc0 + static_cast<uint64_t>((stage * Cfg::STAGE_BYTES) >> 4);
            if (ptx::elect_one()) {
              if (!skip_mma) {
#pragma unroll
                for (int ks = 0; ks < Cfg::KSUB; ++ks) {
                  const uint64_t adesc = adesc_s + static_cast<uint64_t>((ks * 32) >> 4);
                  const uint64_t bdesc = bdesc_s + static_cast<uint64_t>((ks * Cfg::UMMA_K * 128) >> 4);
                  const uint32_t acc = (kk > 0 || ks > 0 || pr.accumulate) ? 1u : 0u;
                  if (ESIZE == 2) ptx::umma_f16_pair(tmem_d, adesc, bdesc, idesc, acc);
                  else ptx::umma_tf32_pair(tmem_d, adesc, bdesc, idesc, acc);
                }
              }
              ptx::umma_commit_pair(&empty_bar[stage], 3);
            }
            __syncwarp();
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            mw_issue += SB200_CLOCK() - ti0;
#ifdef SB200_PROFILE_TRACE
            if (p.prof && lane == 0 && blockIdx.x == 0 && iter == 3 && ps == 0 && kk < 64) {
              p.prof[2048 + kk * 8 + 3] = tw;
              p.prof[2048 + kk * 8 + 4] = ti0;
              p.prof[2048 + kk * 8 + 5] = SB200_CLOCK();
            }
#endif
          }
          if (ok && pr.commit) {
            if (ptx::elect_one()) ptx::umma_commit_pair(&slot_full[slot], 3);
            __syncwarp();
          }
        }
      }
#ifdef SB200_PROFILE
      if (p.prof && lane == 0) {
        p.prof[4096 + pair * 128 + 127] = static_cast<long long>(ptx::globaltimer_ns());  // all MMAs issued
        p.prof[blockIdx.x * 8 + 0] = SB200_CLOCK_LIGHT() - mt0;
        p.prof[blockIdx.x * 8 + 1] = mw_full;
        p.prof[blockIdx.x * 8 + 2] = mw_free;
        p.prof[blockIdx.x * 8 + 5] = mw_issue;
      }
#else
      (void)mw_full; (void)mw_free; (void)mw_issue; (void)mt0;
#endif
    }
#ifdef SB200_PROFILE_TRACE
  } else if (warp == 8 && Cfg::MODE == kPresumNone) {
    // tracing only: an observer that waits on the full barriers in ring order and notes when each completed
    if (lane == 0 && rank == 0 && p.prof) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {   // tracing runs with the static deal only
        const int unit = pair + it * num_pairs;
        if (unit >= total_units(p)) break;
        const WorkUnit wu = unit_of(p, unit);
        for (int ps = 0; ok && ps < nproducts; ++ps)
          for (int kk = 0; kk < wu.k1 - wu.k0; ++kk) {
            if (!ptx::mbar_wait(&full_bar[stage], phase, abort_flag, p.wait_ns)) { ok = false; break; }
            if (blockIdx.x == 0 && it == 3 && ps == 0 && kk < 64) p.prof[2048 + kk * 8 + 2] = clock64();
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
      }
    }
#endif
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue warps (both CTAs, own TMEM half)
    const int quarter = warp & 3;
    uint32_t full_bits = 0;
    uint32_t iter = 0;
    bool ok = true;
    const long long et0 = SB200_CLOCK();
    long long ew_full = 0;
    for (int it = 0; ok; ++it, ++iter, cursor.done(lane)) {
      const int unit = cursor.next(&ok);
      if (unit < 0) break;
      const WorkUnit wu = unit_of(p, unit);
      const TileCoord tile = tile_of(wu.tile, p.tiles_m, p.tiles_n, p.band);
      const uint32_t sx = p.prog.alternate_slots ? (iter & 1u) : 0u;
      for (int es = 0; ok && es < p.prog.nepilogues; ++es) {
        const sb200_epilogue_t& ep = p.prog.epilogue[es];
        const SplitStep sp = split_step(ep, wu.part, wu.nparts);
        if (sp.skip) continue;
        const long long split_tile = static_cast<long long>(wu.split_idx) * 4 + sp.q;
        int* flag = p.split_flags + split_tile * 8 + rank * 4 + quarter;
        float* split_tile_buf = p.split_buf + (split_tile * 2 + rank) * (128 * BN);
        auto wait_slots = [&]() -> bool {
          for (int s0 = 0; s0 < SLOTS; ++s0) {
            if ((ep.wait_full_mask >> s0) & 1u) {
              const uint32_t s = s0 ^ sx;
              const long long tw = SB200_CLOCK();
              const bool got = ptx::mbar_wait_warp<true>(&slot_full[s], (full_bits >> s) & 1u, abort_flag, p.wait_ns);
              ew_full += SB200_CLOCK() - tw;
              if (!got) {
                if (lane == 0) raise_abort(p, abort_flag, kStatusEpilogueTimeout);
                return false;
              }
              full_bits ^= (1u << s);
            }
          }
#ifdef SB200_PROFILE
          const unsigned long long tf0 = ptx::globaltimer_ns();
#endif
          if (sp.add_partial && !wait_flag(flag, p.split_epoch, abort_flag, p.wait_ns)) {
            if (lane == 0) raise_abort(p, abort_flag, kStatusSplitTimeout);
            return false;
          }
#ifdef SB200_PROFILE
          if (p.prof && sp.add_partial && warp == 2 && lane == 0)
            p.prof[blockIdx.x * 8 + 6] += static_cast<long long>(ptx::globaltimer_ns() - tf0);
#endif
          ptx::tc_fence_after_sync();
          return true;
        };
        // hand-off tiles are [32-column chunk][float4 index][128 rows][4]: a column half uses its half of the chunks
        const long long half_off = static_cast<long long>(wu.col_part) * (128 * BN / 2);
        const long long tile_off = (static_cast<long long>(wu.ws_slot) * 2 + rank) * (128 * BN) + half_off;
        const long long outer_off = (static_cast<long long>(wu.tile) * 2 + rank) * (128 * BN) + half_off;
#ifdef SB200_PROFILE_EPILOGUE
        const long long te0 = SB200_CLOCK();
        const long long ew0 = ew_full;
#endif
        ok = epilogue_body<ESIZE, BN, Cfg::NSRC_MAX, Cfg::NSLOT_MAX, Cfg::SCALED>(p.out, p.ldo, (ep.dst & 2) ? p.out_rows2 : p.out_rows,
                                                     (ep.dst & 1) ? p.out_cols2 : p.out_cols, p.ws, ep, sx, tmem_base, quarter,
                                                     lane, tile_off, static_cast<long long>(blockIdx.x) * (128 * BN), outer_off,
                                                     tile.i * Cfg::PAIR_M + static_cast<int>(rank) * Cfg::BM,
                                                     tile.j * BN + wu.col_part * (BN / 2),
                                                     staging + (warp - 2) * kStagingWarpBytes,
                                                     sp.redirect ? split_tile_buf : nullptr,
                                                     sp.add_partial ? split_tile_buf : nullptr,
                                                     SB200_DEBUG_BIT(p, 32), wait_slots, p.alpha, p.beta, p.cin, p.ldc,
                                                     (SB200_PROF_PTR(p) && blockIdx.x == 0 && warp == 2) ? SB200_PROF_PTR(p) + 1190 : nullptr,
                                                     ESIZE == 2 && p.bf16 != 0, (BN / 32) / wu.col_parts);
        if (!ok) break;
#ifdef SB200_PROFILE_EPILOGUE
        if (p.prof && blockIdx.x == 0 && warp == 2 && lane == 0 && es < 16) {
          // per epilogue step: cycles in the body without the slot wait, and the count
          p.prof[1200 + es * 2] += (SB200_CLOCK() - te0) - (ew_full - ew0);
          p.prof[1200 + es * 2 + 1] += 1;
        }
#endif
        if (sp.redirect && !p.drop_split_flags) raise_flag(flag, p.split_epoch, lane);
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          for (int s = 0; s < SLOTS; ++s)
            if ((ep.release_mask >> s) & 1u) ptx::mbar_arrive_cluster(&slot_free[s ^ sx], 0);
        }
      }
    }
#ifdef SB200_PROFILE
    if (p.prof && warp == 2 && lane == 0 && rank == 0)
      p.prof[4096 + pair * 128 + 126] = static_cast<long long>(ptx::globaltimer_ns());  // last epilogue step done
#endif
    (void)ew_full;
    (void)et0;
  } else if (warp >= Cfg::FIRST_PRESUM_WARP) {
    // ------------------------------------------------------------------ presum warps (both CTAs)
    if (Cfg::MODE == kPresumFeed) {
      const int ptid = threadIdx.x - Cfg::FIRST_PRESUM_WARP * 32;
      constexpr int PT = Cfg::PRESUM_WARPS * 32;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = 0; ok; ++it, cursor.done(lane)) {
        const int unit = cursor.next(&ok);
        if (unit < 0) break;
        const WorkUnit wu = unit_of(p, unit);
        const TileCoord tile = tile_of(wu.tile, p.tiles_m, p.tiles_n, p.band);
        const int row0 = tile.i * Cfg::PAIR_M + static_cast<int>(rank) * Cfg::BM;
        const int col0 = tile.j * BN + static_cast<int>(rank) * Cfg::BN_CTA;
        for (int ps = 0; ok && ps < nproducts; ++ps) {
          const sb200_product_t& pr = p.prog.product[ps];
          const bool a_mt = pr.a.nterms > 1;
          const bool b_mt = pr.b.nterms > 1;
          for (int kk = wu.k0; kk < wu.k1; ++kk) {
            bool got = ptx::mbar_wait_cluster(&empty_bar[stage], phase ^ 1u, abort_flag, p.wait_ns);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
              if (lane == 0) raise_abort(p, abort_flag, kStatusPresumTimeout);
              ok = false;
              break;
            }
            const uint32_t sa = ptx::smem_u32(smem + stage * Cfg::STAGE_BYTES);
            const uint32_t sb = sa + Cfg::A_BYTES;
            if (a_mt) build_operand_tile<ESIZE, Cfg::BM, 8, PT, false>(sa, 0u, pr.a, p.view, row0, kk * BK, ptid, p.bf16 != 0);
            if (b_mt)
              build_operand_tile<ESIZE, BK, Cfg::BN_CTA * ESIZE / 16, PT, Cfg::B_SWZ32>(sb, Cfg::BLK_BYTES, pr.b, p.view,
                                                                                        kk * BK, col0, ptid, p.bf16 != 0);
            if (a_mt || b_mt) ptx::fence_proxy_async_all();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(&full_bar[stage], 0);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else if (Cfg::MODE == kPresumJob && !SB200_DEBUG_BIT(p, 16)) {  // bit 4: measurement aid, skip the presum job
      const int ptid = threadIdx.x - Cfg::FIRST_PRESUM_WARP * 32;
      constexpr int PT = Cfg::PRESUM_WARPS * 32;
      if (p.panels.enabled) presum_panels_job<ESIZE, PT>(p, ptid, presum_slot);
      else presum_job<ESIZE>(p, blockIdx.x * PT + ptid, gridDim.x * PT);
    }
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  // neither CTA may leave (and release its shared memory and barriers) while its peer can still signal into it
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace sb200
