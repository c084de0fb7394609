// Module, pass manager and pass registry of the loop IR (see dot_loop_ir.h), plus their C-ABI
// (triton_ext_dot_ir.h).
#include "dot_loop_ir.h"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace {

struct RegisteredPass {
  std::string argument;
  mlir::PassAllocatorFunction make;
};
std::mutex g_reg_mu;
std::vector<RegisteredPass> &registered() {
  static std::vector<RegisteredPass> *v = new std::vector<RegisteredPass>();
  return *v;
}

const char *pred_name(int p) {
  static const char *k[] = {"slt", "sle", "sgt", "sge", "ult", "ule", "ugt", "uge", "eq", "ne"};
  return (p >= 0 && p < 10) ? k[p] : "?";
}

bool eval_pred(int pred, int32_t lhs, int32_t rhs) {
  const uint32_t ul = static_cast<uint32_t>(lhs), ur = static_cast<uint32_t>(rhs);
  switch (pred) {
    case TXIR_SLT: return lhs < rhs;
    case TXIR_SLE: return lhs <= rhs;
    case TXIR_SGT: return lhs > rhs;
    case TXIR_SGE: return lhs >= rhs;
    case TXIR_ULT: return ul < ur;
    case TXIR_ULE: return ul <= ur;
    case TXIR_UGT: return ul > ur;
    case TXIR_UGE: return ul >= ur;
    case TXIR_EQ: return lhs == rhs;
    default: return lhs != rhs;
  }
}

}  // namespace

namespace mlir {

int PassManager::run(ModuleOp &module) {
  int index = 0;
  for (auto &p : passes_) {
    ++index;
    p->module_ = &module;
    p->failed_ = false;
    p->runOnOperation();
    p->module_ = nullptr;
    if (p->failed_) return index;
  }
  return 0;
}

void registerPass(const PassAllocatorFunction &fn) {
  std::unique_ptr<Pass> probe = fn();
  if (!probe) return;
  std::lock_guard<std::mutex> lock(g_reg_mu);
  for (RegisteredPass &r : registered())
    if (r.argument == probe->getArgument()) {
      r.make = fn;
      return;
    }
  registered().push_back(RegisteredPass{probe->getArgument(), fn});
}

}  // namespace mlir

extern "C" {

txir_module *txir_module_create(void) { return new txir_module(); }
void txir_module_destroy(txir_module *m) { delete m; }

int32_t txir_module_add_loop(txir_module *m, const txir_loop *loop) {
  if (!m || !loop) return -1;
  m->loops.push_back(*loop);
  return static_cast<int32_t>(m->loops.size()) - 1;
}

int32_t txir_module_add_dot(txir_module *m, const tx_dot_problem *problem, int32_t block_k) {
  if (!m || !problem || block_k <= 0 || problem->k < 0) return -1;
  txir::DotEntry d;
  d.problem = *problem;
  d.block_k = block_k;
  m->dots.push_back(d);
  const int32_t dot_index = static_cast<int32_t>(m->dots.size()) - 1;
  txir_loop l{};
  l.lo = 0;
  l.hi = problem->k;
  l.step = block_k;
  l.step_is_constant = 1;
  l.has_cmp = 1;
  l.pred = TXIR_SLT;  // k < K_main : operand tiles lie wholly inside [0, K)
  l.iv_operand = 0;
  l.comparand = (problem->k / block_k) * block_k;
  l.comparand_invariant = 1;
  l.fold = TXIR_NOT_FOLDED;
  l.body = TXIR_BODY_DOT;
  l.origin = -1;
  l.dot_index = dot_index;
  m->loops.push_back(l);
  return dot_index;
}

int32_t txir_module_num_loops(const txir_module *m) { return m ? static_cast<int32_t>(m->loops.size()) : 0; }

int32_t txir_module_get_loop(const txir_module *m, int32_t index, txir_loop *out) {
  if (!m || !out || index < 0 || index >= static_cast<int32_t>(m->loops.size())) return -1;
  *out = m->loops[index];
  return 0;
}

int32_t txir_module_set_loop(txir_module *m, int32_t index, const txir_loop *loop) {
  if (!m || !loop || index < 0 || index >= static_cast<int32_t>(m->loops.size())) return -1;
  if (loop->dot_index >= static_cast<int32_t>(m->dots.size())) return -1;
  m->loops[index] = *loop;
  return 0;
}

int32_t txir_module_num_dots(const txir_module *m) { return m ? static_cast<int32_t>(m->dots.size()) : 0; }

int32_t txir_module_get_dot(const txir_module *m, int32_t i, tx_dot_problem *problem, tx_dot_config *config,
                            tx_dot_plan_info *preview) {
  if (!m || i < 0 || i >= static_cast<int32_t>(m->dots.size())) return -1;
  if (problem) *problem = m->dots[i].problem;
  if (config) *config = m->dots[i].config;
  if (preview) *preview = m->dots[i].preview;
  return m->dots[i].lowered ? 1 : 0;
}

int32_t txir_module_set_attr(txir_module *m, const char *key, const char *value) {
  if (!m || !key || !value) return -1;
  m->attrs[key] = value;
  return 0;
}

const char *txir_module_get_attr(const txir_module *m, const char *key) {
  if (!m || !key) return nullptr;
  auto it = m->attrs.find(key);
  return it == m->attrs.end() ? nullptr : it->second.c_str();
}

const char *txir_module_print(txir_module *m) {
  if (!m) return "";
  std::string s = "module {\n";
  char buf[256];
  for (size_t i = 0; i < m->loops.size(); ++i) {
    const txir_loop &l = m->loops[i];
    snprintf(buf, sizeof buf, "  %%loop%zu = scf.for %%iv = %d to %d step %d", i, l.lo, l.hi, l.step);
    s += buf;
    if (l.origin >= 0) {
      snprintf(buf, sizeof buf, " iter_args(<- %%loop%d)", l.origin);
      s += buf;
    }
    s += " {\n";
    if (l.has_cmp) {
      if (l.fold == TXIR_NOT_FOLDED) {
        if (l.iv_operand == 0)
          snprintf(buf, sizeof buf, "    %%c = arith.cmpi %s, %%iv, %d\n", pred_name(l.pred), l.comparand);
        else
          snprintf(buf, sizeof buf, "    %%c = arith.cmpi %s, %d, %%iv\n", pred_name(l.pred), l.comparand);
      } else {
        snprintf(buf, sizeof buf, "    %%c = arith.constant %s\n", l.fold == TXIR_FOLDED_TRUE ? "true" : "false");
      }
      s += buf;
    }
    if (l.body == TXIR_BODY_DOT) {
      const bool folded_true = l.fold == TXIR_FOLDED_TRUE, folded_false = l.fold == TXIR_FOLDED_FALSE;
      s += folded_true ? "    tt.load (unmasked) ; tt.dot\n"
                       : (folded_false ? "    tt.load (masked) ; tt.dot\n" : "    scf.if %c { tt.load } else { tt.load masked } ; tt.dot\n");
    } else {
      s += l.fold == TXIR_FOLDED_TRUE ? "    arith.addf\n"
                                      : (l.fold == TXIR_FOLDED_FALSE ? "    arith.subf\n" : "    scf.if %c { arith.addf } else { arith.subf }\n");
    }
    s += "  }\n";
  }
  for (size_t i = 0; i < m->dots.size(); ++i) {
    const txir::DotEntry &d = m->dots[i];
    snprintf(buf, sizeof buf, "  // dot%zu: m=%d n=%d k=%d BLOCK_K=%d split=%d block_n=%d stages=%d lowered=%d\n", i, d.problem.m,
             d.problem.n, d.problem.k, d.block_k, d.config.k_split_point, d.config.block_n, d.config.stages, (int)d.lowered);
    s += buf;
  }
  s += "}\n";
  m->printed = s;
  return m->printed.c_str();
}

int64_t txir_module_simulate(const txir_module *m, int32_t origin_index) {
  if (!m) return 0;
  int64_t acc = 0;
  for (size_t i = 0; i < m->loops.size(); ++i) {
    const txir_loop &l = m->loops[i];
    if (static_cast<int32_t>(i) != origin_index && l.origin != origin_index) continue;
    if (l.step <= 0) continue;
    for (int64_t iv = l.lo; iv < l.hi; iv += l.step) {
      bool c = true;
      if (l.has_cmp) {
        if (l.fold == TXIR_FOLDED_TRUE) c = true;
        else if (l.fold == TXIR_FOLDED_FALSE) c = false;
        else c = l.iv_operand == 0 ? eval_pred(l.pred, static_cast<int32_t>(iv), l.comparand)
                                   : eval_pred(l.pred, l.comparand, static_cast<int32_t>(iv));
      }
      if (l.body == TXIR_BODY_DOT) acc += c ? 1 : 1000;
      else acc += c ? (iv + 1) : -(iv + 1);
    }
  }
  return acc;
}

TritonExtPassManagerRef txir_pass_manager_create(void) { return new mlir::PassManager(); }
void txir_pass_manager_destroy(TritonExtPassManagerRef pm) { delete pm; }
int32_t txir_pass_manager_size(TritonExtPassManagerRef pm) { return pm ? static_cast<int32_t>(pm->size()) : 0; }
const char *txir_pass_manager_pass_argument(TritonExtPassManagerRef pm, int32_t index) {
  if (!pm || index < 0 || index >= static_cast<int32_t>(pm->size())) return nullptr;
  return pm->at(index).getArgument();
}
int32_t txir_pass_manager_run(TritonExtPassManagerRef pm, txir_module *m) {
  if (!pm || !m) return -1;
  return pm->run(*m);
}
int32_t txir_registered_pass_count(void) {
  std::lock_guard<std::mutex> lock(g_reg_mu);
  return static_cast<int32_t>(registered().size());
}
int32_t txir_registered_pass_lookup(const char *argument) {
  if (!argument) return -1;
  std::lock_guard<std::mutex> lock(g_reg_mu);
  for (size_t i = 0; i < registered().size(); ++i)
    if (registered()[i].argument == argument) return static_cast<int32_t>(i);
  return -1;
}

}  // extern "C"
