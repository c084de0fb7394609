/*
 * triton_ext_loop_split_text.h — LoopSplit over printed Triton IR, exported by the loop_split extension library.
 *
 * The reference's LoopSplit is an MLIR pass (pass/LoopSplit/LoopSplit.cpp:124-196: clone the scf.for, run the
 * first copy over [lo, mid) and the second over [mid, hi), replace the compare of the induction variable by a
 * constant in each). MLIR's C++ API is not available to this library, so the same rewrite is offered on the
 * textual form every Triton tool prints and parses (`tt.func` / `scf.for` / `arith.cmpi` as printed by
 * mlir::Operation::print without locations); the caller parses the result back with its own MLIR context, which
 * verifies it, and canonicalises it (the lit test's `-canonicalize`, pass/LoopSplit/test/loop-split.mlir:1).
 *
 * Accepted loops are the reference's (LoopSplit.cpp:107-144): a positive constant step; an arith.cmpi with
 * predicate slt / sle / sgt / sge or the unsigned forms on the induction variable; the other operand defined
 * outside the loop; the first such compare in the body decides the split. Loops nested in a loop that is not
 * split are looked at too. Constants and definitions are resolved among the lines of the tt.func that holds the loop
 * (SSA names repeat from function to function).
 *
 * Beyond the reference (its LoopSplit.cpp:105 leaves "mask logic" as a TODO), in TXLS_INTENT mode only: a loop with
 * no such scalar compare but with tensor compares of the form
 *     arith.cmpi slt|sle, <expand_dims/broadcast of (tt.splat iv + tt.make_range [0, E))>, <... of tt.splat bound>
 * (the K masks of a tt.dot operand: `k + arange(BLOCK_K) < K`), bound defined outside the loop, is split where those
 * masks stop being all-true (iv + E <= bound): in the first copy every such compare over the same range and bound
 * becomes `arith.constant dense<true>`, which a canonicaliser folds out of the loads; the second copy keeps them.
 * The form of loops that count K blocks is recognised too:
 *     arith.cmpi slt|sle, <... of tt.make_range [0, E)>, <... of tt.splat (bound - iv * c)>,   c a positive constant,
 * all-true while iv * c + E <= bound.
 */
#ifndef TRITON_EXT_LOOP_SPLIT_TEXT_H
#define TRITON_EXT_LOOP_SPLIT_TEXT_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TXLS_API __attribute__((visibility("default")))

typedef enum tx_loop_split_mode {
  /* mid = min(lo + ceildiv(max(T - lo, 0), step) * step, max(hi, lo)), T = comparand (slt, sge) or comparand + 1
   * (sle, sgt); a compare with the induction variable on the right is read with the swapped predicate. Keeps the
   * meaning of the loop for every bound whose distance from lo (plus one, plus a step) stays inside the induction type.
   * Unsigned predicates (ult, ule, ugt, uge) are monotone in the induction variable only while that is non-negative:
   * such a compare is split only when the loop's lower bound is a constant >= 0, and the emitted mid point is
   * guarded at run time: a comparand with its sign bit set (an unsigned value above every non-negative induction
   * value) gives mid = hi, so the whole range stays in the first copy, where the compare has its one value.
   * With any other lower bound an unsigned compare is left alone (the loop may still be split on a later compare). */
  TXLS_INTENT = 0,
  /* Exactly the operations the reference emits (LoopSplit.cpp:147-190): the comparand as mid point, +step / -step
   * for sle / sge, `mid_diff += step - mid_diff % step` when the step is not 1, no clamping, the inverted
   * predicate for a swapped compare. For running the reference's lit test. */
  TXLS_AS_WRITTEN = 1
} tx_loop_split_mode;

/* Rewrites `ir_text` (one module, printed without locations). On success returns 0, stores a malloc'ed,
 * NUL-terminated result in *out_text (release it with tx_loop_split_free) and the number of loops that were
 * split in *loops_split. Returns 1 for invalid arguments and 2 for text whose regions do not balance. */
TXLS_API int tx_loop_split_text(const char *ir_text, int mode, char **out_text, int32_t *loops_split);
TXLS_API void tx_loop_split_free(char *text);

#ifdef __cplusplus
}
#endif
#endif /* TRITON_EXT_LOOP_SPLIT_TEXT_H */
