// loop_split — bisect a loop whose induction variable is compared with a loop-invariant value, so
// that the comparison is constant in each half:  [lo, hi)  ->  [lo, mid) ; [mid, hi).
//
// Re-implements the reference pass pass/LoopSplit/LoopSplit.cpp (argument "triton-loop-split",
// Passes.td:6) on the loop IR of dot_loop_ir.h. For the tt.dot K loop the compare is
// `k < K_main`; the halves are the unpredicated main loop and the masked remainder, and `mid` is
// handed to the kernels as tx_dot_config::k_split_point.
//
// Two modes, chosen by the module attribute "loop_split.mode":
//   "intent" (default)  mid is the first induction value at which the comparison changes, rounded
//                       up to the iteration grid and clamped to [lo, hi]. This is what Passes.td:9-11
//                       describes, and it preserves the meaning of the loop for every predicate.
//   "as-written"        the arithmetic of LoopSplit.cpp:156-193 verbatim, including its quirks
//                       (operand swap done with a logical negation, :51-52; the mid point always
//                       pushed up by 1..step when step != 1, :165-174; unsigned remainder of a
//                       signed difference; no clamping). Kept so that the known answers of the
//                       reference's lit test (test/loop-split.mlir) can be reproduced exactly.
#include <cstdint>
#include <cstring>

#include "dot_loop_ir.h"

namespace {

struct CmpTraits {
  bool valid, greater, equal, is_unsigned;
};

// Same table as LoopSplit.cpp:35-44.
CmpTraits traits(int pred) {
  switch (pred) {
    case TXIR_SGE: return {true, true, true, false};
    case TXIR_SGT: return {true, true, false, false};
    case TXIR_SLE: return {true, false, true, false};
    case TXIR_SLT: return {true, false, false, false};
    case TXIR_UGE: return {true, true, true, true};
    case TXIR_UGT: return {true, true, false, true};
    case TXIR_ULE: return {true, false, true, true};
    case TXIR_ULT: return {true, false, false, true};
    default: return {false, false, false, false};
  }
}

// a < b  <=>  b > a : exchange the operands of a predicate.
int swap_operands(int pred) {
  switch (pred) {
    case TXIR_SLT: return TXIR_SGT;
    case TXIR_SLE: return TXIR_SGE;
    case TXIR_SGT: return TXIR_SLT;
    case TXIR_SGE: return TXIR_SLE;
    case TXIR_ULT: return TXIR_UGT;
    case TXIR_ULE: return TXIR_UGE;
    case TXIR_UGT: return TXIR_ULT;
    case TXIR_UGE: return TXIR_ULE;
    default: return pred;
  }
}

// !(a < b)  <=>  a >= b : what arith::invertPredicate computes (used by LoopSplit.cpp:52).
int negate(int pred) {
  switch (pred) {
    case TXIR_SLT: return TXIR_SGE;
    case TXIR_SLE: return TXIR_SGT;
    case TXIR_SGT: return TXIR_SLE;
    case TXIR_SGE: return TXIR_SLT;
    case TXIR_ULT: return TXIR_UGE;
    case TXIR_ULE: return TXIR_UGT;
    case TXIR_UGT: return TXIR_ULE;
    case TXIR_UGE: return TXIR_ULT;
    case TXIR_EQ: return TXIR_NE;
    default: return TXIR_EQ;
  }
}

int32_t wrap_add(int32_t a, int32_t b) { return static_cast<int32_t>(static_cast<uint32_t>(a) + static_cast<uint32_t>(b)); }
int32_t wrap_sub(int32_t a, int32_t b) { return static_cast<int32_t>(static_cast<uint32_t>(a) - static_cast<uint32_t>(b)); }

struct Split {
  bool ok = false;
  int32_t mid = 0;
  bool greater = false;  // the comparison is false below mid and true from mid on
};

Split split_as_written(const txir_loop &l) {
  Split s;
  int pred = l.pred;
  if (!traits(pred).valid) return s;
  if (l.iv_operand == 1) pred = negate(pred);
  const CmpTraits t = traits(pred);
  int32_t mid = l.comparand;
  if (t.equal) mid = wrap_add(mid, t.greater ? -l.step : l.step);
  if (l.step != 1) {
    int32_t d = wrap_sub(mid, l.lo);
    const uint32_t rem = static_cast<uint32_t>(d) % static_cast<uint32_t>(l.step);
    const int32_t upd = wrap_sub(l.step, static_cast<int32_t>(rem));
    d = wrap_add(d, upd);
    mid = wrap_add(l.lo, d);
  }
  s.ok = true;
  s.mid = mid;
  s.greater = t.greater;
  return s;
}

Split split_intent(const txir_loop &l) {
  Split s;
  int pred = l.pred;
  if (!traits(pred).valid) return s;
  if (l.iv_operand == 1) pred = swap_operands(pred);
  const CmpTraits t = traits(pred);
  int64_t v = l.comparand;
  if (t.is_unsigned) {
    // Unsigned order equals signed order while every induction value is non-negative.
    if (l.lo < 0) return s;
    if (v < 0) v = INT64_MAX / 2;  // 2^31 or more as unsigned: above every induction value
  }
  // First induction value at which the comparison has its late value.
  //   iv <  v : true below v          iv <= v : true below v+1
  //   iv >  v : true from v+1 on      iv >= v : true from v on
  const int64_t flip = (t.greater != t.equal) ? v + 1 : v;
  const int64_t lo = l.lo, hi = l.hi, step = l.step;
  int64_t mid = lo;
  if (flip > lo) mid = lo + (flip - lo + step - 1) / step * step;
  if (mid > hi) mid = hi;
  if (mid < lo) mid = lo;
  s.ok = true;
  s.mid = static_cast<int32_t>(mid);
  s.greater = t.greater;
  return s;
}

struct LoopBisectPass : public mlir::Pass {
  const char *getArgument() const override { return "triton-loop-split"; }
  const char *getDescription() const override { return "Loop splitter"; }

  void runOnOperation() override {
    mlir::ModuleOp &module = getOperation();
    const bool as_written = std::strcmp(module.attr("loop_split.mode", "intent"), "as-written") == 0;
    // Snapshot the loop count: loops created here are not revisited (the reference collects the
    // loops first, then rewrites, LoopSplit.cpp:208-217).
    const size_t n = module.loops.size();
    std::vector<txir_loop> out;
    std::vector<int32_t> new_index(n, -1);   // where old loop i now lives
    std::vector<bool> fresh;                 // out[j] was created by this run (origin already final)
    for (size_t i = 0; i < n; ++i) {
      txir_loop l = module.loops[i];
      new_index[i] = static_cast<int32_t>(out.size());
      const bool candidate = l.step_is_constant && l.step > 0 && l.has_cmp && l.fold == TXIR_NOT_FOLDED &&
                             l.comparand_invariant;
      Split s;
      if (candidate) s = as_written ? split_as_written(l) : split_intent(l);
      if (!s.ok) {
        out.push_back(l);
        fresh.push_back(false);
        continue;
      }
      // Loop 1 keeps the original's place and runs [lo, mid); loop 2 follows it, runs [mid, hi) and
      // takes loop 1's results as its initial values (LoopSplit.cpp:179-185). The compare becomes
      // the constant !greater in loop 1 and greater in loop 2 (:187-193).
      txir_loop first = l, second = l;
      first.hi = s.mid;
      first.fold = s.greater ? TXIR_FOLDED_FALSE : TXIR_FOLDED_TRUE;
      second.lo = s.mid;
      second.fold = s.greater ? TXIR_FOLDED_TRUE : TXIR_FOLDED_FALSE;
      second.origin = static_cast<int32_t>(out.size());
      out.push_back(first);
      fresh.push_back(false);
      out.push_back(second);
      fresh.push_back(true);
      if (l.dot_index >= 0 && l.dot_index < static_cast<int32_t>(module.dots.size()) && !s.greater) {
        // Unmasked-while-true compare: [lo, mid) is the main loop. 0 means "undecided" in
        // tx_dot_config, so a split at 0 is recorded as -1.
        module.dots[l.dot_index].config.k_split_point = s.mid == 0 ? -1 : s.mid;
      }
    }
    for (size_t j = 0; j < out.size(); ++j)
      if (!fresh[j] && out[j].origin >= 0 && out[j].origin < static_cast<int32_t>(n))
        out[j].origin = new_index[out[j].origin];
    module.loops.swap(out);
  }
};

}  // namespace

#include "TritonExtPassGlue.inc"
