// Tile program: the per-output-tile schedule that one CTA of the persistent kernel executes.
//
// It plays the role of the reference project's compile-time schedule vocabulary
// (include/cutlass/gemm/device/strassen_decls.h:145-1922: which presums a kernel reads, which products Mi it
// runs, which +-Mi and interim sources each output sums, which Mi share a launch) but as a small POD table
// that the Python front end emits and the kernel interprets, instead of C++ template instantiations.
//
// A program is a list of PRODUCT steps (executed by the TMA producer, the presum warps and the MMA issuer)
// and a list of EPILOGUE steps (executed by the epilogue warps).  Products accumulate into TMEM slots
// (128 lanes x BN fp32 columns each).  The two sides hand slots back and forth with two credit counters per
// slot, each an mbarrier:
//     slot_full[s]  +1 by a product step with commit = 1 (when its MMAs have completed)
//                   -1 by an epilogue step that lists s in wait_full_mask
//     slot_free[s]  +1 by an epilogue step that lists s in release_mask (when it has finished reading s)
//                   -1 by a product step with wait_free = 1 (before its first MMA touches s)
// slot_free starts with one credit.  Per program and per slot the sequence must alternate
// wait_free, ..., release and commit, ..., wait_full, so that a program can repeat for tile after tile.
#pragma once
#include <stdint.h>

#define SB200_MAX_TERMS 4
#define SB200_MAX_PRODUCTS 8
#define SB200_MAX_EPILOGUES 12
#define SB200_MAX_SLOT_TERMS 3
#define SB200_MAX_SRC_TERMS 3
#define SB200_NUM_VIEWS 16
#define SB200_NUM_WS 20

// Operand view table (index into KernelParams::tmap / ::view):
//   0..3   A quadrants A0,A1,A2,A3 (level 0: view 0 is the whole A)
//   4..7   materialised A presums S1,S2,A02,A1S2
//   8..11  B quadrants B0,B1,B2,B3 (level 0: view 8 is the whole B)
//   12..15 materialised B presums B10,B31,S3,S3B2
// fp32 hand-off buffer table (index into KernelParams::ws).  Every buffer is tile-contiguous and private to the
// CTA that owns the tile.  0..3 belong to the level-1 program itself.  The others connect a level-1 launch to the
// level above it (level 2: the launch computes one quadrant-product of the outer recursion step, and its four
// output quadrants q = 0..3 continue the outer postsum chain):
//   4 + q    outer destination: the launch's output quadrant q kept in fp32 for later launches
//   8 + q    outer source added to output quadrant q
//   12 + q   second outer source, used only by the extra step below
//   16 + q   fp32 destination of the extra step
// An "extra step" is an epilogue step without slots that follows the step writing output quadrant q: it adds
// ws[4 + q] (just written by the same threads) and ws[12 + q] and writes either ws[16 + q] or output quadrant q.
enum {
  SB200_WS_INNER = 0,
  SB200_WS_OUTER_DST = 4,
  SB200_WS_OUTER_SRC = 8,
  SB200_WS_OUTER_SRC2 = 12,
  SB200_WS_EXTRA_DST = 16,
};

enum {
  SB200_VIEW_A0 = 0,
  SB200_VIEW_PA0 = 4,
  SB200_VIEW_B0 = 8,
  SB200_VIEW_PB0 = 12,
};

typedef struct {
  int8_t nterms;                 // 1: one tile, loaded by TMA; 2..4: combined by the presum warps in shared memory
  int8_t view[SB200_MAX_TERMS];  // operand view of each term
  int8_t coef[SB200_MAX_TERMS];  // +1 / -1; evaluated left to right in fp32 (or fp64), rounded once
} sb200_operand_t;

typedef struct {
  sb200_operand_t a, b;
  uint8_t slot;        // TMEM slot the product accumulates into
  uint8_t accumulate;  // 0: first MMA overwrites the slot, 1: continue the sum already in the slot
  uint8_t negate;      // 1: the product enters with a minus sign (A operand negated by the MMA)
  uint8_t wait_free;   // 1: take one slot_free credit before the first MMA
  uint8_t commit;      // 1: give one slot_full credit after the last MMA
  uint8_t pad[3];
} sb200_product_t;

typedef struct {
  uint8_t nslots;
  uint8_t slot[SB200_MAX_SLOT_TERMS];
  int8_t slot_sign[SB200_MAX_SLOT_TERMS];
  uint8_t wait_full_mask;  // slots whose slot_full credit this step takes before reading
  uint8_t release_mask;    // slots that get a slot_free credit when this step is done
  uint8_t nsrc;            // fp32 workspace tiles added to the sum
  uint8_t src[SB200_MAX_SRC_TERMS];
  uint8_t dst_kind;        // 0: output quadrant `dst` in the output type; 1: fp32 workspace buffer `dst`
  uint8_t dst;
  uint8_t pad[2];
} sb200_epilogue_t;

typedef struct {
  int32_t nproducts;
  int32_t nepilogues;
  int32_t alternate_slots;  // 1: XOR every slot id with (tile counter & 1): double buffering for 1-product programs
  int32_t needs_feed;       // 1: some operand has nterms > 1 (needs the presum warps)
  sb200_product_t product[SB200_MAX_PRODUCTS];
  sb200_epilogue_t epilogue[SB200_MAX_EPILOGUES];
  // epilogue step e runs after product step epilogue_after[e] has been issued (documentation / checking only:
  // the epilogue warps simply run their steps in order and block on wait_full_mask)
  uint8_t epilogue_after[SB200_MAX_EPILOGUES];
} sb200_program_t;
