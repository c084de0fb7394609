"""B200-native `tt.dot` tile-GEMM path behind triton-ext's extension API.

Sub-modules:
  backend  - ctypes binding of the `b200_dot` kernels (include/b200_dot.h)
  plugin   - loader harness for the pass-plugin C-ABI (include/triton_ext_plugin.h)
  conf     - `triton-ext.conf` metadata and TRITON_EXT_NAMES gating
  parallel - N-sharded / K-sharded multi-GPU drivers
"""
__all__ = ["backend", "attention", "plugin", "conf", "parallel"]
