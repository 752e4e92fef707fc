// The tile programs the kernels run (level 0, level 1, and level 1 tied into a level-2 run).
//
// Nothing here is written by hand: the tables come from the Python front end, which derives them from the algorithm
// DSL (subcuber_b200/emit.py, subcuber_b200/algos), checks their protocol and algebra
// (subcuber_b200/tile_program.py) and writes them as sw_tile_programs.inc when the library is built
// (subcuber_b200/build.py).  The arithmetic contract is the reference project's
// src/algos/strassen_winograd_level1.py:16-42:
//   S1=A2+A3  S2=S1-A0  A02=A0-A2  A1S2=A1-S2      B10=B1-B0  B31=B3-B1  S3=B31+B0  S3B2=S3-B2
//   M0=A0*B0  M1=A1*B2  M2=S2*S3   M3=A02*B31  M4=S1*B10  M5=A1S2*B3  M6=A3*S3B2
//   C0=M0+M1  C1=M0+M2+M4+M5       C2=M0+M2+M3-M6         C3=M0+M2+M3+M4
// Where the reference emitter copies pre-written sources and only prints its schedule (src/compile.py:48-131,
// 646-653), a new algorithm or plan here is an edit of the DSL side alone.
#pragma once
#include <string.h>

#include "tile_program.h"
#include "sw_tile_programs.inc"

static_assert(SB200_EMITTED_PROGRAM_BYTES == sizeof(sb200_program_t),
              "sw_tile_programs.inc was generated for another layout of sb200_program_t: rebuild");

namespace sb200 {
namespace programs {

// The program called `name` ("level0", "level1_first_early", "level2_m4_launch2", ...); false when there is none.
inline bool find(const char* name, sb200_program_t* out) {
  for (int i = 0; i < SB200_NUM_EMITTED_PROGRAMS; ++i)
    if (strcmp(sb200_emitted_programs[i].name, name) == 0) {
      memcpy(out, sb200_emitted_programs[i].bytes, sizeof(*out));
      return true;
    }
  return false;
}
inline sb200_program_t get(const char* name) {
  sb200_program_t pg;
  if (!find(name, &pg)) memset(&pg, 0, sizeof(pg));  // an empty program: the launch does nothing
  return pg;
}

inline sb200_program_t level0() { return get("level0"); }
// all seven products of a tile in one launch, operand sums formed in shared memory
inline sb200_program_t level1_fused() { return get("level1_full_fly"); }
inline sb200_program_t level1_strassen() { return get("level1_strassen"); }
// Strassen's original algorithm on materialised presums: the program, and the ten presums (five per side) with the
// view slots they are read through
inline sb200_program_t level1_strassen_presum() { return get("level1_strassen_presum"); }
typedef sb200_presum_pair PresumPair;
constexpr int kStrassenPresumsPerSide = 5;
inline const PresumPair* strassen_presums(int side) { return sb200_strassen_presums[side]; }
// the two launches of the interleaved-presum plan
inline sb200_program_t level1_first() { return get("level1_first_early"); }
inline sb200_program_t level1_second() { return get("level1_second_taps"); }
// all seven products in one launch, presums read from the workspace as the launch's presum warps publish them
inline sb200_program_t level1_merged() { return get("level1_merged"); }

// Level 2: the outer recursion step applies the same seven-product scheme to half-size blocks, and each outer product
// is a level-1 GEMM (two launches) whose epilogue steps also carry the outer postsums through three fp32 chain
// buffers X0, X1, X2:
//   m0: X0 = m0 | m1: C0 = X0 + m1 | m2: X1 = X0 + m2 | m4: X2 = m4, X0 = X2 + X1 | m5: C1 = X0 + m5
//   m3: X0 = X1 + m3, C3 = X0 + X2 | m6: C2 = X0 - m6
typedef sb200_level2_child Level2Child;
inline const Level2Child* level2_children() { return sb200_level2_children; }
// launch 1 or 2 of group `child` (0..6, execution order)
inline sb200_program_t level2_launch(int child, int launch) {
  char name[48];
  strcpy(name, "level2_");
  strcat(name, sb200_level2_children[child].name);
  strcat(name, launch == 1 ? "_launch1" : "_launch2");
  return get(name);
}

}  // namespace programs
}  // namespace sb200
