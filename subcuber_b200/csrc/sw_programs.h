// Hand-checked tile programs for level 0 and level 1 (2 TMEM slots of 256 columns, or 4 of 128).
//
// The arithmetic contract is the reference project's src/algos/strassen_winograd_level1.py:16-42:
//   S1=A2+A3  S2=S1-A0  A02=A0-A2  A1S2=A1-S2      B10=B1-B0  B31=B3-B1  S3=B31+B0  S3B2=S3-B2
//   M0=A0*B0  M1=A1*B2  M2=S2*S3   M3=A02*B31  M4=S1*B10  M5=A1S2*B3  M6=A3*S3B2
//   C0=M0+M1  C1=M0+M2+M4+M5       C2=M0+M2+M3-M6         C3=M0+M2+M3+M4
// The same tables are produced by the Python front end (subcuber_b200/emit.py); tests compare the two.
#pragma once
#include <string.h>

#include "tile_program.h"

namespace sb200 {
namespace programs {

enum { A0 = 0, A1 = 1, A2 = 2, A3 = 3, PS1 = 4, PS2 = 5, PA02 = 6, PA1S2 = 7,
       B0 = 8, B1 = 9, B2 = 10, B3 = 11, PB10 = 12, PB31 = 13, PS3 = 14, PS3B2 = 15 };

inline sb200_operand_t term1(int v) {
  sb200_operand_t o;
  memset(&o, 0, sizeof(o));
  o.nterms = 1;
  o.view[0] = (int8_t)v;
  o.coef[0] = 1;
  return o;
}
inline sb200_operand_t terms(int n, const int* v, const int* c) {
  sb200_operand_t o;
  memset(&o, 0, sizeof(o));
  o.nterms = (int8_t)n;
  for (int i = 0; i < n; ++i) {
    o.view[i] = (int8_t)v[i];
    o.coef[i] = (int8_t)c[i];
  }
  return o;
}
// On-the-fly operand combinations, term order chosen so that left-to-right evaluation reproduces the
// reference oracle's expression tree (strassen_reference_l1.cuh:68-75) bit for bit.
inline sb200_operand_t fly_S1() { int v[] = {A2, A3}; int c[] = {1, 1}; return terms(2, v, c); }
inline sb200_operand_t fly_S2() { int v[] = {A2, A3, A0}; int c[] = {1, 1, -1}; return terms(3, v, c); }
inline sb200_operand_t fly_A02() { int v[] = {A0, A2}; int c[] = {1, -1}; return terms(2, v, c); }
inline sb200_operand_t fly_A1S2() { int v[] = {A2, A3, A0, A1}; int c[] = {-1, -1, 1, 1}; return terms(4, v, c); }
inline sb200_operand_t fly_B10() { int v[] = {B1, B0}; int c[] = {1, -1}; return terms(2, v, c); }
inline sb200_operand_t fly_B31() { int v[] = {B3, B1}; int c[] = {1, -1}; return terms(2, v, c); }
inline sb200_operand_t fly_S3() { int v[] = {B3, B1, B0}; int c[] = {1, -1, 1}; return terms(3, v, c); }
inline sb200_operand_t fly_S3B2() { int v[] = {B3, B1, B0, B2}; int c[] = {1, -1, 1, -1}; return terms(4, v, c); }

inline void add_product(sb200_program_t& pg, sb200_operand_t a, sb200_operand_t b, int slot, int accumulate, int negate,
                        int wait_free, int commit) {
  sb200_product_t& p = pg.product[pg.nproducts++];
  memset(&p, 0, sizeof(p));
  p.a = a;
  p.b = b;
  p.slot = (uint8_t)slot;
  p.accumulate = (uint8_t)accumulate;
  p.negate = (uint8_t)negate;
  p.wait_free = (uint8_t)wait_free;
  p.commit = (uint8_t)commit;
  if (a.nterms > 1 || b.nterms > 1) pg.needs_feed = 1;
}

// slots/signs: up to 3 (slot, sign) pairs; srcs: up to 3 workspace ids; masks are bit sets of slot ids.
inline void add_epilogue(sb200_program_t& pg, int nslots, const int* slots, const int* signs, int nsrc, const int* srcs,
                         int wait_mask, int release_mask, int dst_kind, int dst) {
  sb200_epilogue_t& e = pg.epilogue[pg.nepilogues];
  memset(&e, 0, sizeof(e));
  e.nslots = (uint8_t)nslots;
  for (int i = 0; i < nslots; ++i) {
    e.slot[i] = (uint8_t)slots[i];
    e.slot_sign[i] = (int8_t)signs[i];
  }
  e.nsrc = (uint8_t)nsrc;
  for (int i = 0; i < nsrc; ++i) e.src[i] = (uint8_t)srcs[i];
  e.wait_full_mask = (uint8_t)wait_mask;
  e.release_mask = (uint8_t)release_mask;
  e.dst_kind = (uint8_t)dst_kind;
  e.dst = (uint8_t)dst;
  pg.epilogue_after[pg.nepilogues] = (uint8_t)(pg.nproducts - 1);
  pg.nepilogues++;
}

enum { P = 0, Q = 1, mP = 1, mQ = 2 };
// U is dead once C1 is formed, before V is written: they share a buffer (a smaller L2-resident hand-off set)
enum { WS_M0 = 0, WS_M4 = 1, WS_U = 2, WS_V = 2 };

// Level 0: one product per tile, the two (or four) slots used alternately so that the epilogue of tile t
// overlaps the mainloop of tile t+1.
inline sb200_program_t level0() {
  sb200_program_t pg;
  memset(&pg, 0, sizeof(pg));
  pg.alternate_slots = 1;
  add_product(pg, term1(A0), term1(B0), P, 0, 0, 1, 1);
  int s[] = {P}, g[] = {1};
  add_epilogue(pg, 1, s, g, 0, nullptr, mP, mP, 0, 0);
  return pg;
}

// Level 1, all seven products of a tile in one CTA.  `fly` selects where multi-quadrant operands come from:
//   fly = true  : formed on the fly in shared memory by the presum warps (no workspace for operands)
//   fly = false : read from the materialised presum workspace by TMA (views 4..7 and 12..15)
// One fp32 hand-off tile (M4) goes through the workspace; everything else stays in tensor memory.
inline sb200_program_t level1_full(bool fly) {
  sb200_program_t pg;
  memset(&pg, 0, sizeof(pg));
  const int sP[] = {P}, sQ[] = {Q}, sPQ[] = {P, Q}, pos1[] = {1}, pos2[] = {1, 1};
  const int srcM4[] = {WS_M4};
  add_product(pg, term1(A1), term1(B2), Q, 0, 0, 1, 1);                                       // Q  = M1
  add_product(pg, term1(A0), term1(B0), P, 0, 0, 1, 1);                                       // P  = M0
  add_epilogue(pg, 2, sPQ, pos2, 0, nullptr, mP | mQ, mP | mQ, 0, 0);                         // C0 = P + Q
  add_product(pg, fly ? fly_S1() : term1(PS1), fly ? fly_B10() : term1(PB10), Q, 0, 0, 1, 1); // Q  = M4
  add_product(pg, fly ? fly_S2() : term1(PS2), fly ? fly_S3() : term1(PS3), P, 1, 0, 1, 1);   // P += M2  (U)
  add_epilogue(pg, 1, sQ, pos1, 0, nullptr, mQ, mQ, 1, WS_M4);                                // ws[M4] = Q
  add_product(pg, fly ? fly_A1S2() : term1(PA1S2), term1(B3), Q, 1, 0, 1, 1);                 // Q += M5
  add_epilogue(pg, 2, sPQ, pos2, 0, nullptr, mP | mQ, mP | mQ, 0, 1);                         // C1 = U + M4 + M5
  add_product(pg, fly ? fly_A02() : term1(PA02), fly ? fly_B31() : term1(PB31), P, 1, 0, 1, 1); // P += M3 (V2)
  add_epilogue(pg, 1, sP, pos1, 1, srcM4, mP, mP, 0, 3);                                      // C3 = V2 + M4
  add_product(pg, term1(A3), fly ? fly_S3B2() : term1(PS3B2), P, 1, 1, 1, 1);                 // P -= M6
  add_epilogue(pg, 1, sP, pos1, 0, nullptr, mP, mP, 0, 2);                                    // C2 = V2 - M6
  return pg;
}

// Strassen's original algorithm (the second <2,2,2;7> algorithm of this library; the reference names other
// Strassen-like algorithms as future work, README.md:179, and leaves StrassenType::Strassen stubbed,
// include/cutlass/gemm/kernel/strassen_gemm.h:1360-1398):
//   M1=(A0+A3)(B0+B3)  M2=(A2+A3)B0  M3=A0(B1-B3)  M4=A3(B2-B0)  M5=(A0+A1)B3  M6=(A2-A0)(B0+B1)  M7=(A1-A3)(B2+B3)
//   C0=M1+M4-M5+M7     C1=M3+M5      C2=M2+M4      C3=M1-M2+M3+M6
// All seven products of a tile in one CTA, operand sums formed on the fly (no operand has more than two terms).
// Slot P accumulates M1+M7, then M3+M6; slot Q accumulates M4-M5, then holds M2; M1 and M4 are tapped into per-CTA
// fp32 tiles before their slots go on accumulating.
enum { WS_T1 = 1, WS_T4 = 2 };
inline sb200_operand_t pair_of(int v0, int v1, int c1) { int v[] = {v0, v1}; int c[] = {1, c1}; return terms(2, v, c); }
inline sb200_program_t level1_strassen() {
  sb200_program_t pg;
  memset(&pg, 0, sizeof(pg));
  const int sP[] = {P}, sQ[] = {Q}, sPQ[] = {P, Q}, pos1[] = {1}, pos2[] = {1, 1}, posneg[] = {1, -1};
  const int srcT1[] = {WS_T1}, srcT4[] = {WS_T4};
  add_product(pg, pair_of(A0, A3, 1), pair_of(B0, B3, 1), P, 0, 0, 1, 1);    // P  = M1
  add_epilogue(pg, 1, sP, pos1, 0, nullptr, mP, mP, 1, WS_T1);                // ws[T1] = M1
  add_product(pg, term1(A3), pair_of(B2, B0, -1), Q, 0, 0, 1, 1);             // Q  = M4
  add_epilogue(pg, 1, sQ, pos1, 0, nullptr, mQ, mQ, 1, WS_T4);                // ws[T4] = M4
  add_product(pg, pair_of(A1, A3, -1), pair_of(B2, B3, 1), P, 1, 0, 1, 1);    // P += M7
  add_product(pg, pair_of(A0, A1, 1), term1(B3), Q, 1, 1, 1, 1);              // Q -= M5
  add_epilogue(pg, 2, sPQ, pos2, 0, nullptr, mP | mQ, mP, 0, 0);              // C0 = (M1+M7) + (M4-M5)
  add_product(pg, term1(A0), pair_of(B1, B3, -1), P, 0, 0, 1, 1);             // P  = M3
  add_epilogue(pg, 2, sPQ, posneg, 1, srcT4, mP, mP | mQ, 0, 1);              // C1 = M3 - (M4-M5) + M4
  add_product(pg, pair_of(A2, A0, -1), pair_of(B0, B1, 1), P, 1, 0, 1, 1);    // P += M6
  add_product(pg, pair_of(A2, A3, 1), term1(B0), Q, 0, 0, 1, 1);              // Q  = M2
  add_epilogue(pg, 1, sQ, pos1, 1, srcT4, mQ, 0, 0, 2);                       // C2 = M2 + M4
  add_epilogue(pg, 2, sPQ, posneg, 1, srcT1, mP, mP | mQ, 0, 3);              // C3 = (M3+M6) - M2 + M1
  return pg;
}

// Level 1 with interleaved presum, launch 1 of 2: the two products that need no presum; M0 is also handed
// to launch 2 through the fp32 workspace.  The presum warps of this launch materialise the eight presums.
inline sb200_program_t level1_first() {
  sb200_program_t pg;
  memset(&pg, 0, sizeof(pg));
  const int sP[] = {P}, sPQ[] = {P, Q}, pos1[] = {1}, pos2[] = {1, 1};
  add_product(pg, term1(A0), term1(B0), P, 0, 0, 1, 1);                // P = M0
  add_product(pg, term1(A1), term1(B2), Q, 0, 0, 1, 1);                // Q = M1
  add_epilogue(pg, 1, sP, pos1, 0, nullptr, mP, 0, 1, WS_M0);          // ws[M0] = P   (overlaps M1)
  add_epilogue(pg, 2, sPQ, pos2, 0, nullptr, mQ, mP | mQ, 0, 0);       // C0 = P + Q
  return pg;
}

// Launch 1 of 2 with an early release: the copy of M0 to the hand-off tile frees slot P at once and C0 is summed
// from that tile (read back by the threads that wrote it) and slot Q.  The next tile's first product then never
// waits for an epilogue step.  Used when the launch is not tied into a level above (one fp32 source fewer there).
inline sb200_program_t level1_first_early() {
  sb200_program_t pg;
  memset(&pg, 0, sizeof(pg));
  const int sP[] = {P}, sQ[] = {Q}, pos1[] = {1};
  const int srcM0[] = {WS_M0};
  add_product(pg, term1(A0), term1(B0), P, 0, 0, 1, 1);                // P = M0
  add_product(pg, term1(A1), term1(B2), Q, 0, 0, 1, 1);                // Q = M1
  add_epilogue(pg, 1, sP, pos1, 0, nullptr, mP, mP, 1, WS_M0);         // ws[M0] = P   (overlaps M1), P free
  add_epilogue(pg, 1, sQ, pos1, 1, srcM0, mQ, mQ, 0, 0);               // C0 = M0 + Q
  return pg;
}

// Launch 2 of 2: the five products that read presums from the workspace through TMA.
inline sb200_program_t level1_second() {
  sb200_program_t pg;
  memset(&pg, 0, sizeof(pg));
  const int sP[] = {P}, sQ[] = {Q}, sPQ[] = {P, Q}, pos1[] = {1}, pos2[] = {1, 1};
  const int srcM0[] = {WS_M0}, srcM0M4[] = {WS_M0, WS_M4};
  add_product(pg, term1(PS1), term1(PB10), Q, 0, 0, 1, 1);             // Q  = M4
  add_product(pg, term1(PS2), term1(PS3), P, 0, 0, 1, 1);              // P  = M2
  add_epilogue(pg, 1, sQ, pos1, 0, nullptr, mQ, mQ, 1, WS_M4);         // ws[M4] = Q   (overlaps M2)
  add_product(pg, term1(PA1S2), term1(B3), Q, 1, 0, 1, 1);             // Q += M5
  add_epilogue(pg, 2, sPQ, pos2, 1, srcM0, mP | mQ, mP | mQ, 0, 1);    // C1 = M0 + M2 + M4 + M5
  add_product(pg, term1(PA02), term1(PB31), P, 1, 0, 1, 1);            // P += M3
  add_epilogue(pg, 1, sP, pos1, 2, srcM0M4, mP, mP, 0, 3);             // C3 = M0 + M2 + M3 + M4
  add_product(pg, term1(A3), term1(PS3B2), P, 1, 1, 1, 1);             // P -= M6
  add_epilogue(pg, 1, sP, pos1, 1, srcM0, mP, mP, 0, 2);               // C2 = M0 + M2 + M3 - M6
  return pg;
}

// Launch 2 of 2, the plan in use: no product ever waits for an epilogue step that has not had a whole product's
// time to finish.
//   * a slot that keeps accumulating (P: M2, then + M3) is tapped into an fp32 hand-off tile while the OTHER slot's
//     product runs (the tap adds M0, requested before the wait, see epilogue.cuh);
//   * the last product (M6) goes to slot Q instead of being subtracted into P, so the tap of P after M3 overlaps it,
//     and C2 = V - Q is formed from the hand-off tile;
//   * the slot roles swap from tile to tile (alternate_slots), so the next tile's first product takes the slot that
//     was released a whole product earlier.
// No step reads more than two hand-off tiles, which leaves one source free for the level above.
//   hand-offs: M4, U = M0 + M2, V = M0 + (M2 + M3)   (M0 comes from launch 1)
inline sb200_program_t level1_second_taps() {
  sb200_program_t pg;
  memset(&pg, 0, sizeof(pg));
  pg.alternate_slots = 1;
  const int sP[] = {P}, sQ[] = {Q}, pos1[] = {1}, neg1[] = {-1};
  const int srcC1[] = {WS_U, WS_M4}, srcC3[] = {WS_V, WS_M4}, srcM0[] = {WS_M0}, srcV[] = {WS_V};
  add_product(pg, term1(PS1), term1(PB10), Q, 0, 0, 1, 1);             // Q  = M4
  add_product(pg, term1(PS2), term1(PS3), P, 0, 0, 1, 1);              // P  = M2
  add_epilogue(pg, 1, sQ, pos1, 0, nullptr, mQ, mQ, 1, WS_M4);         // ws[M4] = Q             (during M2)
  add_epilogue(pg, 1, sP, pos1, 1, srcM0, mP, mP, 1, WS_U);            // ws[U]  = M0 + P        (during M5)
  add_product(pg, term1(PA1S2), term1(B3), Q, 0, 0, 1, 1);             // Q  = M5
  add_product(pg, term1(PA02), term1(PB31), P, 1, 0, 1, 1);            // P += M3
  add_epilogue(pg, 1, sQ, pos1, 2, srcC1, mQ, mQ, 0, 1);               // C1 = U + M4 + Q        (during M3)
  add_epilogue(pg, 1, sP, pos1, 1, srcM0, mP, mP, 1, WS_V);            // ws[V]  = M0 + P        (during M6)
  add_product(pg, term1(A3), term1(PS3B2), Q, 0, 0, 1, 1);             // Q  = M6
  add_epilogue(pg, 0, nullptr, nullptr, 2, srcC3, 0, 0, 0, 3);         // C3 = V + M4
  add_epilogue(pg, 1, sQ, neg1, 1, srcV, mQ, mQ, 0, 2);                // C2 = V - Q             (during the next M4)
  return pg;
}

// ---------------------------------------------------------------------------------------------------------------
// Level 2: the outer recursion step applies the same seven-product scheme to half-size blocks, and each outer
// product is a level-1 GEMM (two launches) of this library.  The outer postsums are not separate passes: they ride
// on the epilogue steps of the level-1 launches.  `OuterLink` says how one level-1 GEMM is tied into the outer
// chain; `link_outer` rewrites a level-1 program accordingly (hand-off indices: tile_program.h).
struct OuterLink {
  int dst_fp32;  // 1: the four output quadrants stay in fp32 hand-off buffers ws[4 + q] instead of going to out[q]
  int src;       // 1: ws[8 + q] is added to output quadrant q
  int extra;     // 1: also ws[16 + q] = ws[4 + q] + ws[12 + q];  2: also out[q] = ws[4 + q] + ws[12 + q]
  int negate;    // 1: every product enters with a minus sign (the outer product is subtracted)
};

// `launch` is 1 or 2 (first / second launch of the interleaved-presum plan).  All extra steps run in launch 2:
// the one for quadrant 0 (whose sum launch 1 wrote) first, while the epilogue warps wait for the first product.
inline sb200_program_t link_outer(const sb200_program_t& base, const OuterLink& l, int launch) {
  sb200_program_t pg = base;
  pg.nepilogues = 0;
  memset(pg.epilogue, 0, sizeof(pg.epilogue));
  memset(pg.epilogue_after, 0, sizeof(pg.epilogue_after));
  if (l.negate)
    for (int i = 0; i < pg.nproducts; ++i) pg.product[i].negate ^= 1;
  auto push = [&](const sb200_epilogue_t& e, int after) {
    pg.epilogue[pg.nepilogues] = e;
    pg.epilogue_after[pg.nepilogues] = (uint8_t)after;
    pg.nepilogues++;
  };
  auto extra = [&](int q, int after) {
    sb200_epilogue_t e;
    memset(&e, 0, sizeof(e));
    e.nsrc = 2;
    e.src[0] = (uint8_t)(SB200_WS_OUTER_DST + q);
    e.src[1] = (uint8_t)(SB200_WS_OUTER_SRC2 + q);
    e.dst_kind = (uint8_t)(l.extra == 1 ? 1 : 0);
    e.dst = (uint8_t)(l.extra == 1 ? SB200_WS_EXTRA_DST + q : q);
    push(e, after);
  };
  if (launch == 2 && l.extra) extra(0, 0);
  for (int i = 0; i < base.nepilogues; ++i) {
    sb200_epilogue_t e = base.epilogue[i];
    if (e.dst_kind != 0) {
      push(e, base.epilogue_after[i]);
      continue;
    }
    const int q = e.dst;
    if (l.src) e.src[e.nsrc++] = (uint8_t)(SB200_WS_OUTER_SRC + q);
    if (l.dst_fp32) {
      e.dst_kind = 1;
      e.dst = (uint8_t)(SB200_WS_OUTER_DST + q);
    }
    push(e, base.epilogue_after[i]);
    if (launch == 2 && l.extra) extra(q, base.epilogue_after[i]);
  }
  return pg;
}

// The seven level-1 GEMMs of a level-2 run, in execution order.  Operand codes: 0..3 = raw outer quadrant,
// 4..7 = outer presum (A side: S1, S2, A02, A1S2; B side: B10, B31, S3, S3B2).  Outer chain buffers X0, X1, X2
// (fp32, tile-contiguous, one half-size matrix each):
//   M0:           X0 = M0
//   M1:  C0 = X0 + M1
//   M2:           X1 = X0 + M2              (U)
//   M4:           X2 = M4,  X0 = X2 + X1    (U + M4)
//   M5:  C1 = X0 + M5
//   M3:           X0 = X1 + M3,  C3 = X0 + X2
//   M6:  C2 = X0 - M6
struct Level2Child {
  const char* name;
  int a, b;          // operand codes
  OuterLink link;
  int dst, src, src2, extra_dst;  // X buffer ids (-1: none)
  int out_quadrant;               // output quadrant of C written in the output type (-1: none)
};
inline const Level2Child* level2_children() {
  static const Level2Child kChildren[7] = {
      {"m0", 0, 0, {1, 0, 0, 0}, 0, -1, -1, -1, -1},
      {"m1", 1, 2, {0, 1, 0, 0}, -1, 0, -1, -1, 0},
      {"m2", 5, 6, {1, 1, 0, 0}, 1, 0, -1, -1, -1},
      {"m4", 4, 4, {1, 0, 1, 0}, 2, -1, 1, 0, -1},
      {"m5", 7, 3, {0, 1, 0, 0}, -1, 0, -1, -1, 1},
      {"m3", 6, 5, {1, 1, 2, 0}, 0, 1, 2, -1, 3},
      {"m6", 3, 7, {0, 1, 0, 1}, -1, 0, -1, -1, 2},
  };
  return kChildren;
}

}  // namespace programs
}  // namespace sb200
