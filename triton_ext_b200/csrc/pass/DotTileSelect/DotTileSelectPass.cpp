// dot_tile_select — arithmetic-intensity analysis that picks, for every tt.dot in the module, the
// tile shape, pipeline depth, operand roles (swap for skinny m), schedule and raster group of the
// B200 kernels, and records them in the dot's tx_dot_config. Fields a previous pass or the user has
// already set (for instance loop_split's k_split_point) are kept.
//
// The reference has no such pass; it is registered through the same glue as loop_split so that it
// loads, enumerates and is added to a pipeline the way any triton-ext pass is
// (infra/pass/TritonExtPass.cpp:21-39 of the reference).
//
// Module attribute "dot_tile_select.sm_count" overrides the SM count (default 148).
#include <cstdlib>

#include "dot_loop_ir.h"
#include "dot_tile_model.h"

namespace {

struct DotTileSelectPass : public mlir::Pass {
  const char *getArgument() const override { return "triton-dot-tile-select"; }
  const char *getDescription() const override { return "Pick tcgen05 tile shape and pipeline depth per tt.dot"; }

  void runOnOperation() override {
    mlir::ModuleOp &module = getOperation();
    txd::MachineModel mm;
    const int sm = std::atoi(module.attr("dot_tile_select.sm_count", "148"));
    if (sm > 0) mm.sm_count = sm;
    for (txir::DotEntry &d : module.dots) {
      if (d.problem.m <= 0 || d.problem.n <= 0 || d.problem.k <= 0) continue;
      txd::TileChoice tc;
      const char *why = "";
      if (txd::select_tiles(d.problem, &d.config, mm, tc, &why) != 0) {
        module.attrs["dot_tile_select.error"] = why;
        signalPassFailure();
        return;
      }
      d.config.block_n = tc.block_n;
      d.config.stages = tc.stages;
      d.config.swap_ab = tc.swap_ab ? 1 : 2;
      d.config.schedule = tc.schedule;
      d.config.group_m = tc.group_m;
      d.config.cta_pair = tc.cta_pair ? 1 : 2;
      d.config.atoms = tc.atoms;
      txd::fill_plan_info(d.problem, tc, &d.preview);
    }
  }
};

}  // namespace

#include "TritonExtPassGlue.inc"
