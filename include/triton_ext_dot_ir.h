/*
 * triton_ext_dot_ir.h — C-ABI of the loop IR and pass pipeline that stand where MLIR stands in the
 * reference.
 *
 * The reference's extensions are MLIR passes run by an mlir::PassManager over a ModuleOp
 * (pass/LoopSplit/Passes.td:6 anchors the pass on mlir::ModuleOp; LoopSplit.cpp:204-219 walks its
 * scf.for ops). MLIR is not part of this repository, and the only IR the hot path needs is the loop
 * that LoopSplit rewrites: an scf.for with integer bounds and a constant step whose induction
 * variable is compared with a loop-invariant value (LoopSplit.cpp:107-144), and whose body is the
 * tt.dot tile update. This header models exactly that:
 *
 *   txir_module        ~ mlir::ModuleOp   : an ordered list of loops
 *   txir_loop          ~ scf.for          : [lo, hi) step s, compare sites on the IV, a region tag
 *   mlir::PassManager  ~ mlir::PassManager: an ordered list of passes (see triton_ext_plugin.h)
 *
 * All values are concrete 32-bit integers (the reference's loops are i32, LoopSplit.cpp:160).
 */
#ifndef TRITON_EXT_DOT_IR_H
#define TRITON_EXT_DOT_IR_H

#include <stdint.h>

#include "b200_dot.h"
#include "triton_ext_plugin.h"

#ifdef __cplusplus
extern "C" {
#endif

#define TXIR_API __attribute__((visibility("default")))

/* arith.cmpi predicates. The first eight are the ones LoopSplit accepts (LoopSplit.cpp:35-44). */
typedef enum txir_pred {
  TXIR_SLT = 0, TXIR_SLE = 1, TXIR_SGT = 2, TXIR_SGE = 3,
  TXIR_ULT = 4, TXIR_ULE = 5, TXIR_UGT = 6, TXIR_UGE = 7,
  TXIR_EQ = 8, TXIR_NE = 9
} txir_pred;

/* How a compare site reads after a pass folded it. */
typedef enum txir_fold {
  TXIR_NOT_FOLDED = 0, /* still evaluated every iteration */
  TXIR_FOLDED_FALSE = 1,
  TXIR_FOLDED_TRUE = 2
} txir_fold;

/* What the loop body is. */
typedef enum txir_body {
  TXIR_BODY_SELECT_ADD_SUB = 0, /* the lit-test body: acc = cmp ? acc + x : acc - x
                                   (pass/LoopSplit/test/loop-split.mlir:18-31) */
  TXIR_BODY_DOT = 1             /* acc = tt.dot(A[:, iv:iv+BK], B[iv:iv+BK, :], acc); operand loads
                                   are unmasked where the compare is true, masked otherwise */
} txir_body;

typedef struct txir_loop {
  int32_t lo, hi, step;      /* scf.for bounds; step_is_constant = 0 models a non-constant step */
  int32_t step_is_constant;
  int32_t has_cmp;           /* an arith.cmpi uses the induction variable */
  int32_t pred;              /* txir_pred as written in the IR */
  int32_t iv_operand;        /* 0: cmpi pred, %iv, %v    1: cmpi pred, %v, %iv */
  int32_t comparand;         /* value of %v */
  int32_t comparand_invariant; /* %v is defined outside the loop */
  int32_t fold;              /* txir_fold */
  int32_t body;              /* txir_body */
  int32_t origin;            /* index of the loop this one was split from, or -1 */
  int32_t dot_index;         /* which dot problem the loop belongs to, or -1 */
  int32_t reserved;
} txir_loop;

typedef struct txir_module txir_module;

TXIR_API txir_module *txir_module_create(void);
TXIR_API void txir_module_destroy(txir_module *m);
/* Append a loop; returns its index or -1. */
TXIR_API int32_t txir_module_add_loop(txir_module *m, const txir_loop *loop);
/* Append the canonical K loop of a tt.dot GEMM:  for k in [0, K) step block_k, with the compare
 * `k < (K / block_k) * block_k` guarding the unmasked operand loads. block_k is the BLOCK_K of the
 * source program (a multiple of the kernels' physical K block). Returns the dot index or -1. */
TXIR_API int32_t txir_module_add_dot(txir_module *m, const tx_dot_problem *problem, int32_t block_k);
TXIR_API int32_t txir_module_num_loops(const txir_module *m);
TXIR_API int32_t txir_module_get_loop(const txir_module *m, int32_t index, txir_loop *out);
/* Replace loop `index`, e.g. to give the K loop of a dot the compare the source program really has
 * (its own split point instead of the canonical floor(K / block_k) * block_k). Returns 0 or -1. */
TXIR_API int32_t txir_module_set_loop(txir_module *m, int32_t index, const txir_loop *loop);
TXIR_API int32_t txir_module_num_dots(const txir_module *m);
/* The problem of dot `dot_index`, and the kernel configuration the passes have attached so far
 * (zero fields = not decided). After `loop_split` has run, config->k_split_point is the mid point. */
TXIR_API int32_t txir_module_get_dot(const txir_module *m, int32_t dot_index, tx_dot_problem *problem,
                                     tx_dot_config *config, tx_dot_plan_info *preview);
/* String attributes steer passes, e.g. ("loop_split.mode", "intent" | "as-written"),
 * ("dot_tile_select.sm_count", "148"). Returns 0 on success. */
TXIR_API int32_t txir_module_set_attr(txir_module *m, const char *key, const char *value);
TXIR_API const char *txir_module_get_attr(const txir_module *m, const char *key);
/* Human-readable dump (borrowed pointer, valid until the next call on this module). */
TXIR_API const char *txir_module_print(txir_module *m);
/* Execute loop `index` and the loops split from it in order on a scalar stand-in for the body
 * (acc starts at 0; SELECT_ADD_SUB adds/subtracts iv+1; DOT counts unmasked and masked iterations
 * as acc += 1 / acc += 1000). Used to check that a transformation kept the meaning. */
TXIR_API int64_t txir_module_simulate(const txir_module *m, int32_t origin_index);

/* The pipeline object behind mlir::PassManager*. */
TXIR_API TritonExtPassManagerRef txir_pass_manager_create(void);
TXIR_API void txir_pass_manager_destroy(TritonExtPassManagerRef pm);
TXIR_API int32_t txir_pass_manager_size(TritonExtPassManagerRef pm);
TXIR_API const char *txir_pass_manager_pass_argument(TritonExtPassManagerRef pm, int32_t index);
/* Run every pass in order; returns 0, or the 1-based index of the pass that failed. */
TXIR_API int32_t txir_pass_manager_run(TritonExtPassManagerRef pm, txir_module *m);
/* Number of passes made known through tritonRegisterPluginPass (mlir::registerPass stand-in),
 * and a lookup by command-line argument such as "triton-loop-split". */
TXIR_API int32_t txir_registered_pass_count(void);
TXIR_API int32_t txir_registered_pass_lookup(const char *argument);

/* Implemented by the backend extension library (libb200_dot.so): build a launchable plan from a dot
 * that the `b200_dot` pass has lowered. Returns a tx_dot_status. */
TXIR_API int32_t txir_module_create_plan(const txir_module *m, int32_t dot_index, tx_dot_plan **out_plan);

#ifdef __cplusplus
}
#endif
#endif /* TRITON_EXT_DOT_IR_H */
