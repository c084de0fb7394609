/*
 * TEST INFRASTRUCTURE — not part of the product path.
 *
 * Plain-C restatement of the split-point arithmetic of the reference's LoopSplit pass,
 * pass/LoopSplit/LoopSplit.cpp, exactly as written there (including its quirks), on concrete i32
 * values. It is the checker for the product's `loop_split` extension in "as-written" mode.
 *
 * Followed line by line:
 *   LoopSplit.cpp:35-44   predicate table: {s,u}{ge,gt,le,lt} -> (greater, equal)
 *   LoopSplit.cpp:49-54   induction variable as operand #1 -> arith::invertPredicate (logical negation)
 *   LoopSplit.cpp:107-123 a compare qualifies only if its other operand is defined outside the loop
 *   LoopSplit.cpp:128-138 the step must be a positive constant
 *   LoopSplit.cpp:156-162 mid = comparand; if "equal": mid += greater ? -step : +step   (i32)
 *   LoopSplit.cpp:165-174 if step != 1: d = mid - lo; d += step - (d remui step); mid = lo + d
 *   LoopSplit.cpp:179-185 loop 1 = [lo, mid), loop 2 = [mid, hi), chained through iter_args
 *   LoopSplit.cpp:187-193 compare := !greater in loop 1, greater in loop 2
 *
 * Pinned by tests/test_loop_split.py against the five cases of
 * pass/LoopSplit/test/loop-split.mlir (loop order, folded branch, the -1 / +1 adjust constants).
 */
#include <stdint.h>

enum { LS_SLT = 0, LS_SLE = 1, LS_SGT = 2, LS_SGE = 3, LS_ULT = 4, LS_ULE = 5, LS_UGT = 6, LS_UGE = 7 };

typedef struct ls_result {
  int32_t split;        /* 1 if the loop is bisected */
  int32_t mid;          /* upper bound of loop 1 = lower bound of loop 2 */
  int32_t cmp_in_loop1; /* constant the compare is replaced with in loop 1 (0/1) */
  int32_t cmp_in_loop2;
} ls_result;

static int ls_valid(int pred) { return pred >= LS_SLT && pred <= LS_UGE; }
static int ls_greater(int pred) { return pred == LS_SGT || pred == LS_SGE || pred == LS_UGT || pred == LS_UGE; }
static int ls_equal(int pred) { return pred == LS_SLE || pred == LS_SGE || pred == LS_ULE || pred == LS_UGE; }

/* arith::invertPredicate: the predicate of the negated comparison. */
static int ls_invert(int pred) {
  switch (pred) {
    case LS_SLT: return LS_SGE;
    case LS_SLE: return LS_SGT;
    case LS_SGT: return LS_SLE;
    case LS_SGE: return LS_SLT;
    case LS_ULT: return LS_UGE;
    case LS_ULE: return LS_UGT;
    case LS_UGT: return LS_ULE;
    default: return LS_ULT;
  }
}

static int32_t add32(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }
static int32_t sub32(int32_t a, int32_t b) { return (int32_t)((uint32_t)a - (uint32_t)b); }

__attribute__((visibility("default")))
int ls_bisect_as_written(int32_t lo, int32_t hi, int32_t step, int32_t step_is_constant, int32_t pred,
                         int32_t iv_operand, int32_t comparand, int32_t comparand_invariant, ls_result *out) {
  (void)hi; /* the reference never looks at the upper bound when it picks the mid point */
  out->split = 0;
  out->mid = 0;
  out->cmp_in_loop1 = out->cmp_in_loop2 = 0;
  if (!step_is_constant || step <= 0) return 0;
  if (!ls_valid(pred)) return 0;
  if (iv_operand == 1) pred = ls_invert(pred);
  if (!comparand_invariant) return 0;
  int32_t mid = comparand;
  if (ls_equal(pred)) mid = add32(mid, ls_greater(pred) ? -step : step);
  if (step != 1) {
    int32_t d = sub32(mid, lo);
    uint32_t rem = (uint32_t)d % (uint32_t)step;
    int32_t upd = sub32(step, (int32_t)rem);
    d = add32(d, upd);
    mid = add32(lo, d);
  }
  out->split = 1;
  out->mid = mid;
  out->cmp_in_loop1 = !ls_greater(pred);
  out->cmp_in_loop2 = ls_greater(pred);
  return 1;
}

/* Reference semantics of the ORIGINAL loop, for checking what a split preserved: runs
 * for (iv = lo; iv < hi; iv += step) acc += cmp(iv) ? (iv+1) : -(iv+1). */
__attribute__((visibility("default")))
int64_t ls_run_original(int32_t lo, int32_t hi, int32_t step, int32_t pred, int32_t iv_operand, int32_t comparand) {
  int64_t acc = 0;
  if (step <= 0) return 0;
  for (int64_t iv = lo; iv < hi; iv += step) {
    int32_t a = iv_operand == 0 ? (int32_t)iv : comparand;
    int32_t b = iv_operand == 0 ? comparand : (int32_t)iv;
    int c;
    switch (pred) {
      case LS_SLT: c = a < b; break;
      case LS_SLE: c = a <= b; break;
      case LS_SGT: c = a > b; break;
      case LS_SGE: c = a >= b; break;
      case LS_ULT: c = (uint32_t)a < (uint32_t)b; break;
      case LS_ULE: c = (uint32_t)a <= (uint32_t)b; break;
      case LS_UGT: c = (uint32_t)a > (uint32_t)b; break;
      default: c = (uint32_t)a >= (uint32_t)b; break;
    }
    acc += c ? (iv + 1) : -(iv + 1);
  }
  return acc;
}
