/*
 * triton_ext_plugin.h — the pass-plugin C-ABI of triton-ext, re-implemented.
 *
 * Replaces, symbol for symbol, the reference's infra/pass/TritonExtPassInfra.h:11-26 (declarations)
 * and infra/pass/TritonExtPassInfra.cpp:7-52 (definitions):
 *
 *   tritonAddPluginPass          TritonExtPassInfra.h:11-12   .cpp:19-26
 *   tritonRegisterPluginPass     TritonExtPassInfra.h:14-15   .cpp:28-35
 *   tritonEnumeratePluginPasses  TritonExtPassInfra.h:17-18   .cpp:37-52
 *   TritonExtLoadPass            TritonExtPassInfra.h:24-26   .cpp:7-14
 *
 * The reference takes TRITON_PLUGIN_API / TritonPluginResult / TP_SUCCESS / TP_GENERIC_FAILURE from
 * upstream Triton's "triton/Tools/PluginUtils.h" (TritonExtPassInfra.h:8), which is part of neither
 * the reference nor this repository. The definitions below stand in for it: a two-value result enum
 * whose success value is zero, and an export macro written in return-type position. If the real
 * header is on the include path, define TRITON_EXT_USE_UPSTREAM_PLUGIN_UTILS to use it instead.
 *
 * `mlir::PassManager *` is an opaque handle at this boundary. In this repository it points to the
 * pipeline object declared in triton_ext_dot_ir.h (a pass list over the tt.dot loop IR); built
 * against real MLIR it would be MLIR's own class. C callers see `void *`.
 *
 * Differences from the reference, on purpose:
 *   - tritonEnumeratePluginPasses fills names[0..count-1]; the reference never advances its index
 *     (TritonExtPassInfra.cpp:47-50) and leaves every name in slot 0.
 *   - the registry is guarded by a mutex; the reference's maps are unsynchronised.
 *   - a NULL passName is answered with TP_GENERIC_FAILURE instead of a crash.
 */
#ifndef TRITON_EXT_PLUGIN_H
#define TRITON_EXT_PLUGIN_H

#include <stdint.h>

#ifdef TRITON_EXT_USE_UPSTREAM_PLUGIN_UTILS
#include "triton/Tools/PluginUtils.h"
#else
typedef enum TritonPluginResult {
  TP_SUCCESS = 0,
  TP_GENERIC_FAILURE = 1
} TritonPluginResult;
#ifdef __cplusplus
#define TRITON_PLUGIN_API extern "C" __attribute__((visibility("default"))) TritonPluginResult
#else
#define TRITON_PLUGIN_API __attribute__((visibility("default"))) TritonPluginResult
#endif
#endif

#ifdef __cplusplus
namespace mlir {
class PassManager;
}
typedef mlir::PassManager *TritonExtPassManagerRef;
#else
typedef void *TritonExtPassManagerRef;
#endif

/* Append the pass registered under `passName` to the pipeline `pm`. Unknown name: failure. */
TRITON_PLUGIN_API
tritonAddPluginPass(TritonExtPassManagerRef pm, const char *passName);

/* Make the pass known to the process-wide pass registry (command-line style lookup by argument). */
TRITON_PLUGIN_API
tritonRegisterPluginPass(const char *passName);

/* Two-call protocol: (&n, NULL) reports the count; (&n, names) also fills a caller-owned array of
 * at least n entries with borrowed strings that live as long as the extension library. */
TRITON_PLUGIN_API
tritonEnumeratePluginPasses(uint32_t *passCount, const char **passNames);

/* Called by each extension library from a static initialiser at dlopen time. */
typedef void (*TritonExtRegisterPassFunc)(void);
typedef void (*TritonExtAddPassFunc)(TritonExtPassManagerRef);

TRITON_PLUGIN_API
TritonExtLoadPass(const char *passName, TritonExtRegisterPassFunc registerFunc,
                  TritonExtAddPassFunc addFunc);

#endif /* TRITON_EXT_PLUGIN_H */
