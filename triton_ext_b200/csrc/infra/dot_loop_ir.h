// The loop IR and pass pipeline that extensions in this repository are written against.
//
// It plays the part MLIR plays for the reference's extensions: `mlir::Pass`, `mlir::PassManager`,
// `mlir::registerPass` keep their names so that an extension source here reads like
// pass/LoopSplit/LoopSplit.cpp + infra/pass/TritonExtPass.cpp do there, but the module is the small
// loop list described in triton_ext_dot_ir.h instead of a ModuleOp.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "triton_ext_dot_ir.h"

namespace txir {

struct DotEntry {
  tx_dot_problem problem{};
  tx_dot_config config{};       // fields decided so far by passes (0 = undecided)
  tx_dot_plan_info preview{};   // filled by dot_tile_select / b200_dot
  int32_t block_k = 0;          // BLOCK_K of the source program
  bool lowered = false;         // b200_dot has accepted it
};

}  // namespace txir

// Definition of the opaque C handle.
struct txir_module {
  std::vector<txir_loop> loops;
  std::vector<txir::DotEntry> dots;
  std::map<std::string, std::string> attrs;
  std::string printed;

  const char *attr(const char *key, const char *dflt) const {
    auto it = attrs.find(key);
    return it == attrs.end() ? dflt : it->second.c_str();
  }
};

namespace mlir {

using ModuleOp = ::txir_module;

// One transformation over a module. Mirrors the slice of mlir::Pass the reference uses:
// getArgument() is the command-line name from Passes.td, runOnOperation() does the work.
class Pass {
public:
  virtual ~Pass() = default;
  virtual const char *getArgument() const = 0;
  virtual const char *getDescription() const { return ""; }
  virtual void runOnOperation() = 0;

  ModuleOp &getOperation() { return *module_; }
  void signalPassFailure() { failed_ = true; }

private:
  friend class PassManager;
  ModuleOp *module_ = nullptr;
  bool failed_ = false;
};

class PassManager {
public:
  void addPass(std::unique_ptr<Pass> pass) { passes_.push_back(std::move(pass)); }
  size_t size() const { return passes_.size(); }
  const Pass &at(size_t i) const { return *passes_[i]; }
  // Returns 0, or the 1-based index of the first pass that signalled failure.
  int run(ModuleOp &module);

private:
  std::vector<std::unique_ptr<Pass>> passes_;
};

using PassAllocatorFunction = std::function<std::unique_ptr<Pass>()>;
// Process-wide registry keyed by the pass argument (what `triton-opt -<argument>` would look up).
__attribute__((visibility("default"))) void registerPass(const PassAllocatorFunction &fn);

}  // namespace mlir
