"""Compiler half of the Triton backend that sends a ``@triton.jit`` K-loop kernel to the library GEMM.

Triton finds a backend as a package holding ``compiler.py`` (one ``BaseBackend`` subclass) and
``driver.py`` (one ``DriverBase`` subclass), listed in the ``triton.backends`` entry-point group
(triton 3.6.0 backends/__init__.py:57-62; the interface is backends/compiler.py:23-68). This module is
that ``compiler.py``. Its stages are

    ttir    Triton's own target-independent clean-up of the front end's IR (inliner, canonicaliser,
            combine, CSE), the IR the reference's LoopSplit pass runs on
    b200dot ttir.match_dot_kernel(): the proof that the kernel is one tt.dot K loop, serialised as JSON

The "binary" handed to the launcher is that JSON, not machine code: the machine code is the tcgen05
kernel inside libb200_dot.so, picked per launch by the loop_split / dot_tile_select / b200_dot passes.
A kernel that is not the K loop fails to compile with the reason (ttir.NotCanonical); nothing falls back
to Triton's own code generation.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from types import ModuleType
from typing import Any, Dict, Optional, Tuple

from triton._C.libtriton import ir, passes
from triton.backends.compiler import BaseBackend, GPUTarget, Language

from . import ttir as _ttir

TARGET_NAME = "b200dot"


@dataclass(frozen=True)
class B200DotOptions:
    # The launch options the JIT front end reads from every backend's option object.
    num_warps: int = 4
    num_ctas: int = 1
    num_stages: int = 3
    warp_size: int = 32
    enable_fp_fusion: bool = True
    launch_cooperative_grid: bool = False
    launch_pdl: bool = False
    extern_libs: Optional[tuple] = None
    debug: bool = False
    sanitize_overflow: bool = False
    arch: str = "sm100"
    backend_name: str = TARGET_NAME
    instrumentation_mode: str = ""
    supported_fp8_dtypes: Tuple[str, ...] = ("fp8e4nv", "fp8e5")
    deprecated_fp8_dot_operand_dtypes: Tuple[str, ...] = ()
    default_dot_input_precision: str = "ieee"
    allowed_dot_input_precisions: Tuple[str, ...] = ("ieee", "tf32")
    max_num_imprecise_acc_default: int = 0

    def hash(self) -> str:
        key = "_".join(f"{k}-{v}" for k, v in sorted(self.__dict__.items()))
        return hashlib.sha256(key.encode()).hexdigest()


def _min_dot_size(lhs_type, rhs_type):
    return (1, 1, 32) if lhs_type.scalar.primitive_bitwidth == 8 else (1, 1, 16)


class B200DotBackend(BaseBackend):
    binary_ext = TARGET_NAME

    @staticmethod
    def supports_target(target: GPUTarget) -> bool:
        return target.backend == TARGET_NAME

    def __init__(self, target: GPUTarget) -> None:
        super().__init__(target)
        self.binary_ext = TARGET_NAME

    def hash(self) -> str:
        # Part of Triton's cache key: a proof written by another version of the matcher must not be reused.
        with open(_ttir.__file__, "rb") as f:
            matcher = hashlib.sha256(f.read()).hexdigest()[:16]
        return f"{TARGET_NAME}-{self.target.arch}-{matcher}"

    def parse_options(self, opts: dict) -> Any:
        known = B200DotOptions.__dataclass_fields__.keys()
        return B200DotOptions(**{k: opts[k] for k in known if k in opts and opts[k] is not None})

    def pack_metadata(self, metadata):
        return (metadata.num_warps, metadata.num_ctas, metadata.shared)

    def get_codegen_implementation(self, options) -> dict:
        return {"min_dot_size": _min_dot_size}

    def get_module_map(self) -> Dict[str, ModuleType]:
        return {}

    def load_dialects(self, ctx) -> None:
        pass

    def add_stages(self, stages: dict, options: Any, language: Language = Language.TRITON) -> None:
        if language != Language.TRITON:
            raise RuntimeError("the b200dot backend lowers Triton kernels only")
        stages["ttir"] = lambda src, metadata: self.make_ttir(src, metadata, options)
        stages["ttsplit"] = lambda src, metadata: self.make_loop_split(src, metadata, options)
        stages[TARGET_NAME] = lambda src, metadata: self.make_match(src, metadata, options)

    @staticmethod
    def make_ttir(mod, metadata: dict, options: Any):
        pm = ir.pass_manager(mod.context)
        pm.enable_debug()
        passes.common.add_inliner(pm)
        passes.ttir.add_rewrite_tensor_pointer(pm)
        passes.common.add_canonicalizer(pm)
        passes.ttir.add_combine(pm)
        passes.ttir.add_reorder_broadcast(pm)
        passes.common.add_cse(pm)
        passes.common.add_symbol_dce(pm)
        pm.run(mod, "make_ttir")
        return mod

    @staticmethod
    def make_loop_split(mod, metadata: dict, options: Any):
        """LoopSplit on the kernel's own IR (loop_split_ir.split_loops), parsed back and canonicalised by
        Triton's MLIR context so that each half keeps only the arm of the scf.if its constant compare selects."""
        import os
        import tempfile

        from . import loop_split_ir

        text = str(mod)
        _, args, _ = _ttir.parse_module(text)
        metadata["arg_names"] = [src for _, src, _ in args]
        new_text, n_split = loop_split_ir.split_loops(text)
        metadata["loops_split"] = n_split
        if n_split == 0:
            return mod
        fd, path = tempfile.mkstemp(suffix=".ttir")
        try:
            with os.fdopen(fd, "w") as f:
                f.write(new_text)
            split = ir.parse_mlir_module(path, mod.context)
        finally:
            os.unlink(path)
        split.context = mod.context
        pm = ir.pass_manager(split.context)
        pm.enable_debug()
        passes.common.add_canonicalizer(pm)
        passes.common.add_cse(pm)
        passes.common.add_canonicalizer(pm)
        pm.run(split, "loop_split_cleanup")
        return split

    @staticmethod
    def make_match(mod, metadata: dict, options: Any) -> bytes:
        match = _ttir.match_dot_kernel(str(mod), metadata.get("arg_names"))
        metadata["name"] = match.kernel
        metadata["shared"] = 0
        metadata["num_warps"] = options.num_warps
        metadata["global_scratch_size"] = 0
        metadata["global_scratch_align"] = 1
        metadata["profile_scratch_size"] = 0
        metadata["profile_scratch_align"] = 1
        return match.to_json().encode()


def lower_to_ttir(fn, signature: dict, constexprs: Optional[dict] = None, split: bool = False,
                  arg_names_out: Optional[list] = None) -> str:
    """Front end + the ``ttir`` stage for one specialisation of a ``@triton.jit`` function; needs no GPU.

    `signature` maps every parameter to its Triton type string ("*bf16", "i32", "fp32", "constexpr").
    """
    from triton.compiler import ASTSource

    target = GPUTarget(TARGET_NAME, 100, 32)
    backend = B200DotBackend(target)
    options = backend.parse_options({})
    src = ASTSource(fn, signature, constexprs or {})
    context = ir.context()
    ir.load_dialects(context)
    mod = src.make_ir(target, options, backend.get_codegen_implementation(options), backend.get_module_map(), context)
    mod = backend.make_ttir(mod, {}, options)
    if split:
        meta: dict = {}
        mod = backend.make_loop_split(mod, meta, options)
        if arg_names_out is not None:
            arg_names_out.extend(meta["arg_names"])
    return str(mod)


def analyse(fn, signature: dict, constexprs: Optional[dict] = None, split: bool = True) -> "_ttir.DotKernelMatch":
    """The compile pipeline without a launch: front end, `ttir`, LoopSplit on the IR (`split`), the K-loop match."""
    names: list = []
    text = lower_to_ttir(fn, signature, constexprs, split=split, arg_names_out=names)
    return _ttir.match_dot_kernel(text, names or None)
