"""Loader harness for the pass-plugin C-ABI (include/triton_ext_plugin.h, include/triton_ext_dot_ir.h).

Upstream Triton loads triton-ext extensions by dlopen'ing the libraries named in
``TRITON_PASS_PLUGIN_PATH`` and calling the exported ``tritonEnumeratePluginPasses`` /
``tritonRegisterPluginPass`` / ``tritonAddPluginPass`` (reference README.md:114-121; the symbols are
declared in infra/pass/TritonExtPassInfra.h:11-26). The Triton wheel installed next to this package
has no such loader, so this module plays that part: it loads extension libraries, drives the four
entry points, owns the pipeline object that stands behind ``mlir::PassManager *`` and the loop-IR
module the passes transform.
"""
from __future__ import annotations

import ctypes
import os
from typing import Iterable, Optional

from . import conf
from .backend import Config, PlanInfo, Problem, _LIB_DIR

TP_SUCCESS = 0
TP_GENERIC_FAILURE = 1

TXIR_SLT, TXIR_SLE, TXIR_SGT, TXIR_SGE, TXIR_ULT, TXIR_ULE, TXIR_UGT, TXIR_UGE, TXIR_EQ, TXIR_NE = range(10)
TXIR_NOT_FOLDED, TXIR_FOLDED_FALSE, TXIR_FOLDED_TRUE = 0, 1, 2
TXIR_BODY_SELECT_ADD_SUB, TXIR_BODY_DOT = 0, 1

PRED_BY_NAME = {"slt": 0, "sle": 1, "sgt": 2, "sge": 3, "ult": 4, "ule": 5, "ugt": 6, "uge": 7, "eq": 8, "ne": 9}


class Loop(ctypes.Structure):
    _fields_ = [
        ("lo", ctypes.c_int32), ("hi", ctypes.c_int32), ("step", ctypes.c_int32),
        ("step_is_constant", ctypes.c_int32), ("has_cmp", ctypes.c_int32), ("pred", ctypes.c_int32),
        ("iv_operand", ctypes.c_int32), ("comparand", ctypes.c_int32),
        ("comparand_invariant", ctypes.c_int32), ("fold", ctypes.c_int32), ("body", ctypes.c_int32),
        ("origin", ctypes.c_int32), ("dot_index", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]

    def as_dict(self) -> dict:
        return {n: getattr(self, n) for n, _ in self._fields_ if n != "reserved"}


def make_loop(lo: int, hi: int, step: int, pred: str | int, comparand: int, *, iv_operand: int = 0,
              invariant: bool = True, step_is_constant: bool = True, body: int = TXIR_BODY_SELECT_ADD_SUB) -> Loop:
    l = Loop()
    l.lo, l.hi, l.step = lo, hi, step
    l.step_is_constant = int(step_is_constant)
    l.has_cmp = 1
    l.pred = PRED_BY_NAME[pred] if isinstance(pred, str) else int(pred)
    l.iv_operand = iv_operand
    l.comparand = comparand
    l.comparand_invariant = int(invariant)
    l.fold = TXIR_NOT_FOLDED
    l.body = body
    l.origin = -1
    l.dot_index = -1
    return l


_infra = None
_loaded: dict[str, ctypes.CDLL] = {}


def infra_path() -> str:
    return os.path.join(_LIB_DIR, "libTritonExtPassInfra.so")


def infra() -> ctypes.CDLL:
    """The one registry library of the process (RTLD_GLOBAL so extension libraries bind to it)."""
    global _infra
    if _infra is not None:
        return _infra
    p = infra_path()
    if not os.path.exists(p):
        raise ImportError(f"{p} is missing: run triton_ext_b200.build.build_all() first")
    lib = ctypes.CDLL(p, mode=ctypes.RTLD_GLOBAL)
    vp, i32, cstr = ctypes.c_void_p, ctypes.c_int32, ctypes.c_char_p
    lib.tritonAddPluginPass.argtypes = [vp, cstr]
    lib.tritonRegisterPluginPass.argtypes = [cstr]
    lib.tritonEnumeratePluginPasses.argtypes = [ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(cstr)]
    lib.TritonExtLoadPass.argtypes = [cstr, vp, vp]
    for n in ("tritonAddPluginPass", "tritonRegisterPluginPass", "tritonEnumeratePluginPasses", "TritonExtLoadPass"):
        getattr(lib, n).restype = ctypes.c_int
    lib.txir_module_create.restype = vp
    lib.txir_module_destroy.argtypes = [vp]
    lib.txir_module_add_loop.argtypes = [vp, ctypes.POINTER(Loop)]
    lib.txir_module_add_loop.restype = i32
    lib.txir_module_add_dot.argtypes = [vp, ctypes.POINTER(Problem), i32]
    lib.txir_module_add_dot.restype = i32
    lib.txir_module_num_loops.argtypes = [vp]
    lib.txir_module_num_loops.restype = i32
    lib.txir_module_get_loop.argtypes = [vp, i32, ctypes.POINTER(Loop)]
    lib.txir_module_get_loop.restype = i32
    lib.txir_module_set_loop.argtypes = [vp, i32, ctypes.POINTER(Loop)]
    lib.txir_module_set_loop.restype = i32
    lib.txir_module_num_dots.argtypes = [vp]
    lib.txir_module_num_dots.restype = i32
    lib.txir_module_get_dot.argtypes = [vp, i32, ctypes.POINTER(Problem), ctypes.POINTER(Config), ctypes.POINTER(PlanInfo)]
    lib.txir_module_get_dot.restype = i32
    lib.txir_module_set_attr.argtypes = [vp, cstr, cstr]
    lib.txir_module_set_attr.restype = i32
    lib.txir_module_get_attr.argtypes = [vp, cstr]
    lib.txir_module_get_attr.restype = cstr
    lib.txir_module_print.argtypes = [vp]
    lib.txir_module_print.restype = cstr
    lib.txir_module_simulate.argtypes = [vp, i32]
    lib.txir_module_simulate.restype = ctypes.c_int64
    lib.txir_pass_manager_create.restype = vp
    lib.txir_pass_manager_destroy.argtypes = [vp]
    lib.txir_pass_manager_size.argtypes = [vp]
    lib.txir_pass_manager_size.restype = i32
    lib.txir_pass_manager_pass_argument.argtypes = [vp, i32]
    lib.txir_pass_manager_pass_argument.restype = cstr
    lib.txir_pass_manager_run.argtypes = [vp, vp]
    lib.txir_pass_manager_run.restype = i32
    lib.txir_registered_pass_count.restype = i32
    lib.txir_registered_pass_lookup.argtypes = [cstr]
    lib.txir_registered_pass_lookup.restype = i32
    _infra = lib
    return lib


def load_plugin(path: str) -> ctypes.CDLL:
    """dlopen one extension library; its static initialiser registers the pass (TritonExtLoadPass)."""
    infra()
    path = os.path.abspath(path)
    if path not in _loaded:
        _loaded[path] = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    return _loaded[path]


def plugin_path(name: str) -> str:
    """Where build.py puts the library of extension `name` (its triton-ext.conf name)."""
    return os.path.join(_LIB_DIR, f"lib{name}.so")


def load_plugins_from_env(value: Optional[str] = None) -> list[str]:
    """Load every library listed in TRITON_PASS_PLUGIN_PATH (':' separated), as upstream Triton does."""
    value = os.environ.get("TRITON_PASS_PLUGIN_PATH", "") if value is None else value
    loaded = []
    for p in [v for v in value.split(":") if v]:
        load_plugin(p)
        loaded.append(p)
    return loaded


def load_default_plugins(names: Optional[Iterable[str]] = None) -> list[str]:
    """Load the extensions built in this package, honouring TRITON_EXT_NAMES."""
    allow = list(names) if names is not None else conf.ext_names_filter()
    out = []
    for n in ("loop_split", "dot_tile_select", "b200_dot"):
        if allow and n not in allow:
            continue
        load_plugin(plugin_path(n))
        out.append(n)
    return out


def enumerate_passes() -> list[str]:
    """The two-call protocol of tritonEnumeratePluginPasses."""
    lib = infra()
    n = ctypes.c_uint32(0)
    if lib.tritonEnumeratePluginPasses(ctypes.byref(n), None) != TP_SUCCESS:
        raise RuntimeError("tritonEnumeratePluginPasses failed")
    if n.value == 0:
        return []
    names = (ctypes.c_char_p * n.value)()
    if lib.tritonEnumeratePluginPasses(ctypes.byref(n), names) != TP_SUCCESS:
        raise RuntimeError("tritonEnumeratePluginPasses failed")
    return [names[i].decode() for i in range(n.value)]


def register_pass(name: str) -> int:
    return infra().tritonRegisterPluginPass(name.encode())


def registered_pass_lookup(argument: str) -> int:
    return infra().txir_registered_pass_lookup(argument.encode())


class PassManager:
    """The pipeline object handed to tritonAddPluginPass as `mlir::PassManager *`."""

    def __init__(self):
        self._lib = infra()
        self._h = ctypes.c_void_p(self._lib.txir_pass_manager_create())

    def add(self, name: str) -> int:
        """tritonAddPluginPass(pm, name) -> TritonPluginResult."""
        return self._lib.tritonAddPluginPass(self._h, name.encode())

    def arguments(self) -> list[str]:
        n = self._lib.txir_pass_manager_size(self._h)
        return [self._lib.txir_pass_manager_pass_argument(self._h, i).decode() for i in range(n)]

    def run(self, module: "Module") -> int:
        return self._lib.txir_pass_manager_run(self._h, module._h)

    def __del__(self):
        try:
            if self._h:
                self._lib.txir_pass_manager_destroy(self._h)
                self._h = None
        except Exception:
            pass


class Module:
    """The loop-IR module (stand-in for mlir::ModuleOp)."""

    def __init__(self):
        self._lib = infra()
        self._h = ctypes.c_void_p(self._lib.txir_module_create())

    def add_loop(self, loop: Loop) -> int:
        return self._lib.txir_module_add_loop(self._h, ctypes.byref(loop))

    def add_dot(self, problem: Problem, block_k: int) -> int:
        return self._lib.txir_module_add_dot(self._h, ctypes.byref(problem), block_k)

    def loops(self) -> list[dict]:
        out = []
        for i in range(self._lib.txir_module_num_loops(self._h)):
            l = Loop()
            self._lib.txir_module_get_loop(self._h, i, ctypes.byref(l))
            out.append(l.as_dict())
        return out

    def set_loop(self, index: int, loop: Loop) -> int:
        return self._lib.txir_module_set_loop(self._h, index, ctypes.byref(loop))

    def dot(self, index: int = 0) -> tuple[Problem, Config, dict, bool]:
        pr, cfg, info = Problem(), Config(), PlanInfo()
        rc = self._lib.txir_module_get_dot(self._h, index, ctypes.byref(pr), ctypes.byref(cfg), ctypes.byref(info))
        if rc < 0:
            raise IndexError(index)
        return pr, cfg, info.as_dict(), bool(rc)

    def set_attr(self, key: str, value: str) -> None:
        self._lib.txir_module_set_attr(self._h, key.encode(), value.encode())

    def get_attr(self, key: str) -> Optional[str]:
        v = self._lib.txir_module_get_attr(self._h, key.encode())
        return v.decode() if v is not None else None

    def simulate(self, origin: int) -> int:
        return int(self._lib.txir_module_simulate(self._h, origin))

    def __str__(self) -> str:
        return self._lib.txir_module_print(self._h).decode()

    def __del__(self):
        try:
            if self._h:
                self._lib.txir_module_destroy(self._h)
                self._h = None
        except Exception:
            pass


DEFAULT_PIPELINE = ("loop_split", "dot_tile_select", "b200_dot")


def lower_dot(problem: Problem, block_k: int, pipeline: Iterable[str] = DEFAULT_PIPELINE,
              attrs: Optional[dict] = None, split_comparand: Optional[int] = None) -> tuple[Config, dict, Module]:
    """Run the extension pipeline over one tt.dot K loop and return the kernel configuration it
    produced (split point from loop_split, tiles from dot_tile_select, accepted by b200_dot).
    `split_comparand` is the value the source program compares its induction variable with
    (`k < split_comparand` guards the unmasked loads); default: the last multiple of block_k in K."""
    load_default_plugins()
    m = Module()
    for k, v in (attrs or {}).items():
        m.set_attr(k, str(v))
    if m.add_dot(problem, block_k) < 0:
        raise ValueError("txir_module_add_dot rejected the problem")
    if split_comparand is not None:
        l = Loop()
        m._lib.txir_module_get_loop(m._h, 0, ctypes.byref(l))
        l.comparand = int(split_comparand)
        if m.set_loop(0, l) != 0:
            raise ValueError("txir_module_set_loop rejected the loop")
    pm = PassManager()
    for name in pipeline:
        if pm.add(name) != TP_SUCCESS:
            raise RuntimeError(f"tritonAddPluginPass: unknown pass {name!r}")
    failed = pm.run(m)
    if failed:
        why = m.get_attr("b200_dot.error") or m.get_attr("dot_tile_select.error") or ""
        raise RuntimeError(f"pass #{failed} ({pm.arguments()[failed - 1]}) failed: {why}")
    _, cfg, info, _ = m.dot(0)
    return cfg, info, m
