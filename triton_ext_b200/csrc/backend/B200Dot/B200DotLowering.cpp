// b200_dot — the backend extension's pass: accepts every tt.dot of the module for the sm_100a
// kernels, or fails the pipeline with a reason. It fills whatever kernel configuration earlier passes
// left undecided and marks the dot as lowered; txir_module_create_plan() then turns a lowered dot into
// a launchable tx_dot_plan.
//
// This is what occupies the reference's empty backend slot (backend/CMakeLists.txt, 0 bytes). It is
// registered through the same glue as the pass extensions (reference: infra/pass/TritonExtPass.cpp).
#include <cstdlib>
#include <string>

#include "b200_dot.h"
#include "dot_loop_ir.h"
#include "dot_tile_model.h"

namespace {

struct B200DotLoweringPass : public mlir::Pass {
  const char *getArgument() const override { return "triton-b200-dot"; }
  const char *getDescription() const override { return "Lower tt.dot K loops to B200 tcgen05 kernels"; }

  void fail(mlir::ModuleOp &module, const std::string &why) {
    module.attrs["b200_dot.error"] = why;
    signalPassFailure();
  }

  void runOnOperation() override {
    mlir::ModuleOp &module = getOperation();
    const int sm = std::atoi(module.attr("dot_tile_select.sm_count", "148"));
    for (size_t i = 0; i < module.dots.size(); ++i) {
      txir::DotEntry &d = module.dots[i];
      d.lowered = false;
      if (d.problem.m == 0 || d.problem.n == 0 || d.problem.k == 0) {  // nothing for the tensor pipe
        d.lowered = true;
        continue;
      }
      const int es = txd::elem_bytes(d.problem.ab_dtype);
      if (es != 1 && es != 2) return fail(module, "operand dtype must be f16, bf16, f8e4m3 or f8e5m2");
      const int bk = 128 / es;  // physical K block of the kernels
      // The source loop's BLOCK_K need not match the kernels' physical K block (128 bytes of K).
      // A split point inside a physical block is moved down to the block's start: the remainder
      // loop only adds masking, so letting it absorb whole blocks never changes a result.
      int split = d.config.k_split_point;
      const int last_full = (d.problem.k / bk) * bk;
      if (split > last_full)
        return fail(module, "k_split_point " + std::to_string(split) + " puts a partial K block (K=" +
                                std::to_string(d.problem.k) + ") into the unmasked main loop");
      if (split > 0) {
        split = (split / bk) * bk;
        d.config.k_split_point = split == 0 ? -1 : split;
      }
      tx_dot_plan_info info;
      if (tx_dot_plan_preview(&d.problem, &d.config, sm, &info) != TXD_OK) return fail(module, tx_dot_last_error());
      d.config.block_n = info.block_n;
      d.config.stages = info.stages;
      d.config.swap_ab = info.swap_ab ? 1 : 2;
      d.config.schedule = info.schedule;
      d.config.group_m = info.group_m;
      d.config.cta_pair = info.cta_pair ? 1 : 2;
      d.config.atoms = info.block_k / bk;
      d.preview = info;
      d.lowered = true;
    }
  }
};

}  // namespace

extern "C" __attribute__((visibility("default"))) int32_t txir_module_create_plan(const txir_module *m, int32_t dot_index,
                                                                                  tx_dot_plan **out_plan) {
  if (!m || !out_plan || dot_index < 0 || dot_index >= static_cast<int32_t>(m->dots.size())) return TXD_ERR_INVALID;
  const txir::DotEntry &d = m->dots[dot_index];
  if (!d.lowered) return TXD_ERR_INVALID;  // run the b200_dot pass first
  return tx_dot_plan_create(&d.problem, &d.config, out_plan);
}

#include "TritonExtPassGlue.inc"
