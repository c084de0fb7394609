"""LoopSplit on real Triton IR (text level): bisect an ``scf.for`` whose induction variable is compared with a
loop-invariant value, so that the compare is a constant in each half.

This is the transformation of the reference's pass (pass/LoopSplit/LoopSplit.cpp:124-196): the loop is cloned,
the first copy runs [lo, mid), the second [mid, hi) with the first copy's results as its initial values, and the
compare is replaced by ``true`` in one copy and ``false`` in the other; a canonicalisation afterwards (the lit
test's ``-canonicalize``, pass/LoopSplit/test/loop-split.mlir:1) removes the dead ``scf.if`` arms. Accepted loops
are the reference's (:107-144): a positive constant step, an ``arith.cmpi`` with predicate slt / sle / sgt / sge
(or their unsigned forms) on the induction variable, the other operand defined outside the loop; the first such
compare decides the split.

The mid point is computed so that the split keeps the meaning of the loop for every bound (the reference's
arithmetic adds one whole step when the distance is already a multiple of the step and does not clamp to the
loop's range; see the loop_split extension's "intent" mode, which this follows):

    T   = C for  iv < C / iv >= C,   C + 1 for  iv <= C / iv > C
    mid = min(lo + ceildiv(max(T - lo, 0), step) * step, max(hi, lo))

There are no MLIR C++ headers to build a pass against in this environment, so the rewrite works on the printed IR
and the result is checked by parsing it back with Triton's own MLIR context (compiler.B200DotBackend.make_loop_split).

The rewrite itself is C++ in the loop_split extension library, next to the pass it belongs to
(csrc/pass/LoopSplit/LoopSplitText.cpp, include/triton_ext_loop_split_text.h); this module strips the locations
from the printed module and calls it.
"""
from __future__ import annotations

import ctypes

from .ttir import strip_locations

MODES = {"intent": 0, "as-written": 1}
_lib = None


def _library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        from .. import plugin

        lib = plugin.load_plugin(plugin.plugin_path("loop_split"))
        lib.tx_loop_split_text.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                           ctypes.POINTER(ctypes.c_int32)]
        lib.tx_loop_split_text.restype = ctypes.c_int
        lib.tx_loop_split_free.argtypes = [ctypes.c_void_p]
        lib.tx_loop_split_free.restype = None
        _lib = lib
    return _lib


def split_loops(text: str, mode: str = "intent") -> tuple:
    """Bisect every eligible loop of the printed module. Returns (new text, number of loops split).

    mode "intent" keeps the loop's meaning for every bound (above). mode "as-written" emits exactly the
    reference's operations (LoopSplit.cpp:147-190): the comparand itself as the mid point, plus or minus one step
    for sle / sge, rounded by `mid_diff += step - mid_diff % step` when the step is not 1, no clamping, a compare
    with the induction variable on the right read with the inverted (not the swapped) predicate. It exists so that
    the reference's own lit test can be run against this rewrite; kernels are compiled with "intent"."""
    if mode not in MODES:
        raise ValueError(mode)
    lib = _library()
    out = ctypes.c_void_p()
    n = ctypes.c_int32(0)
    rc = lib.tx_loop_split_text(strip_locations(text).encode(), MODES[mode], ctypes.byref(out), ctypes.byref(n))
    if rc != 0:
        raise ValueError("tx_loop_split_text: " + {1: "invalid arguments", 2: "unbalanced regions in the IR text"}.get(rc, str(rc)))
    try:
        return ctypes.string_at(out).decode(), int(n.value)
    finally:
        lib.tx_loop_split_free(out)
