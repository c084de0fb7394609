"""Driver half of the Triton backend: launches a matched K-loop kernel on the library's tcgen05 GEMM.

Triton's run time asks its active driver for the target (which selects compiler.py's backend), for a
loader that turns the compiled "binary" into a function handle, and for a launcher that is called with
the grid, the stream and the kernel's arguments (triton 3.6.0 compiler/compiler.py:430-466 and
runtime/jit.py:695-746; interface backends/driver.py:13-49). Here the binary is the JSON proof written by
compiler.py; the launcher binds it to the arguments of the launch (ttir.bind), runs the loop_split /
dot_tile_select / b200_dot passes over the resulting tt.dot loop, and calls tx_dot_run on the caller's
stream. There is no other path: a launch the proof does not cover raises, a missing library raises.

The driver never reports itself active, so that installing the package's entry point does not take
Triton's stock CUDA driver away (Triton allows one active driver). Use :func:`activate`.
"""
from __future__ import annotations

from typing import Any

from triton.backends.compiler import GPUTarget
from triton.backends.driver import DriverBase

from . import ttir as _ttir
from .compiler import TARGET_NAME

_TORCH_DTYPES = {"f16": "float16", "bf16": "bfloat16", "f32": "float32", "f8e4m3": "float8_e4m3fn",
                 "f8e5m2": "float8_e5m2"}


class B200DotUtils:
    """What the run time asks the driver about devices and binaries."""

    def get_device_properties(self, device: int) -> dict:
        import torch

        p = torch.cuda.get_device_properties(device)
        return {"max_shared_mem": 232448, "max_num_regs": 65536, "multiprocessor_count": p.multi_processor_count,
                "warpSize": 32, "sm_clock_rate": 0, "mem_clock_rate": 0, "mem_bus_width": 0}

    def load_binary(self, name: str, kernel: bytes, shared: int, device: int) -> tuple:
        """(module, function, registers, spills, max threads): module and function are the match."""
        match = _ttir.DotKernelMatch.from_json(kernel.decode())
        return match, match, 0, 0, 1024


def _integer_argument(values: dict, name: str) -> int:
    """An integer kernel argument, or a field of a host tensor descriptor (<arg>__shape<d>, <arg>__stride<d>)."""
    if name in values:
        return int(values[name])
    arg, _, field = name.rpartition("__")
    desc = values[arg]
    kind, d = field.rstrip("0123456789"), int(field[len(field.rstrip("0123456789")):])
    return int((desc.shape if kind == "shape" else desc.strides)[d])


def _tensor_of(value: Any) -> Any:
    """The tensor behind a kernel argument: the argument itself, or the base of a host tensor descriptor."""
    return value.base if hasattr(value, "base") and hasattr(value, "block_shape") else value


class B200DotLauncher:
    """Called as launcher(gridX, gridY, gridZ, stream, function, metadata..., hooks..., *kernel args)."""

    MAX_CACHED_SHAPES = 256

    def __init__(self, src: Any, metadata: Any):
        self.arg_names = list(src.fn.arg_names)
        self._bound: dict = {}
        self.launches = 0

    def prepare(self, match: _ttir.DotKernelMatch, values: dict, grid: tuple, device: int = 0) -> dict:
        """Bind one launch and run the pass pipeline over its K loop; touches no GPU. Cached per launch shape."""
        import torch

        from .. import backend, plugin

        scalars = {n: _integer_argument(values, n) for n in match.int_args}
        alpha_arg = values.get(match.alpha) if match.alpha in values else None
        key = (tuple(sorted(scalars.items())), tuple(grid), alpha_arg, device)
        entry = self._bound.get(key)
        if entry is None:
            bound = _ttir.bind(match, scalars, grid, {match.alpha: alpha_arg} if alpha_arg is not None else None)
            layouts = {"row": backend.TXD_ROW_MAJOR, "col": backend.TXD_COL_MAJOR}
            problem = backend.make_problem(
                bound.m, bound.n, bound.k, getattr(torch, _TORCH_DTYPES[match.ab_dtype]),
                getattr(torch, _TORCH_DTYPES[match.out_dtype]), a_layout=layouts[bound.a_layout],
                b_layout=layouts[bound.b_layout], lda=bound.lda, ldb=bound.ldb, ldc=bound.ldc, alpha=bound.alpha,
                row_scale=(match.col_scale_arg if bound.swapped else match.row_scale_arg) is not None,
                col_scale=(match.row_scale_arg if bound.swapped else match.col_scale_arg) is not None)
            # The library's K blocks are 128 bytes of K wide; a source block may be narrower. Whole source blocks
            # past the last whole library block belong to the library's masked remainder block.
            phys = 128 // {"f8e4m3": 1, "f8e5m2": 1}.get(match.ab_dtype, 2)
            split = min(bound.k_main, (bound.k // phys) * phys)
            config, info, module = plugin.lower_dot(problem, bound.block_k, split_comparand=split)
            entry = {"bound": bound, "problem": problem, "config": config, "info": info, "ir": str(module), "plan": None}
            if len(self._bound) >= self.MAX_CACHED_SHAPES:  # oldest launch shape goes, with its plan
                old = self._bound.pop(next(iter(self._bound)))
                if old["plan"] is not None:
                    old["plan"].close()
            self._bound[key] = entry
        return entry

    def __call__(self, grid_x: int, grid_y: int, grid_z: int, stream: int, function: Any, packed_metadata: Any,
                 launch_metadata: Any, enter_hook: Any, exit_hook: Any, *args: Any) -> None:
        import ctypes

        import torch

        from .. import backend

        match: _ttir.DotKernelMatch = function
        values = dict(zip(self.arg_names, args))
        a, b, c = (_tensor_of(values[n]) for n in (match.a_arg, match.b_arg, match.c_arg))
        for t, name, dt in ((a, match.a_arg, match.ab_dtype), (b, match.b_arg, match.ab_dtype), (c, match.c_arg, match.out_dtype)):
            if not hasattr(t, "data_ptr") or not t.is_cuda:
                raise TypeError(f"{name} must be a CUDA tensor; there is no CPU path")
            if t.dtype != getattr(torch, _TORCH_DTYPES[dt]):
                raise TypeError(f"{name} is {t.dtype}, the kernel was compiled for {dt}")
        scales = []
        for name in (match.row_scale_arg, match.col_scale_arg):
            t = values[name] if name is not None else None
            if t is not None and not (hasattr(t, "data_ptr") and t.is_cuda and t.dtype == torch.float32):
                raise TypeError(f"{name} must be a CUDA float32 tensor")
            scales.append(t.data_ptr() if t is not None else None)
        entry = self.prepare(match, values, (grid_x, grid_y, grid_z), torch.cuda.current_device())
        if entry["plan"] is None:
            entry["plan"] = backend.DotPlan(entry["problem"], entry["config"])
        plan = entry["plan"]
        if enter_hook is not None:
            enter_hook(launch_metadata)
        ab_size, c_size = a.element_size(), c.element_size()
        if entry["bound"].swapped:  # column-major C: the library's A is the kernel's B (offsets were exchanged by bind)
            a, b, scales = b, a, scales[::-1]
        for off_a, off_b, off_c in entry["bound"].batches or [(0, 0, 0)]:  # one library launch per matrix product
            backend._check(plan._lib.tx_dot_run(plan._h, a.data_ptr() + off_a * ab_size, b.data_ptr() + off_b * ab_size,
                                                c.data_ptr() + off_c * c_size, scales[0], scales[1],
                                                ctypes.c_void_p(int(stream))))
            self.launches += 1
        if exit_hook is not None:
            exit_hook(launch_metadata)

    def lowered_ir(self) -> list:
        """The loop IR after the passes, one text per distinct launch shape (for inspection and tests)."""
        return [e["ir"] for e in self._bound.values()]


class B200DotDriver(DriverBase):

    def __init__(self):
        import torch

        super().__init__()
        self.utils = B200DotUtils()
        self.launcher_cls = B200DotLauncher
        self.get_current_device = torch.cuda.current_device
        self.set_current_device = torch.cuda.set_device
        self.get_device_capability = torch.cuda.get_device_capability
        self.get_current_stream = lambda idx: torch.cuda.current_stream(idx).cuda_stream

    @classmethod
    def is_active(cls) -> bool:
        return False

    def get_current_target(self) -> GPUTarget:
        major, minor = self.get_device_capability(self.get_current_device())
        if major != 10:
            raise RuntimeError(f"the b200dot backend needs an sm_100 device, found sm_{major}{minor}")
        return GPUTarget(TARGET_NAME, major * 10 + minor, 32)

    def get_active_torch_device(self):
        import torch

        return torch.device("cuda", self.get_current_device())

    def get_device_interface(self):
        import torch

        return torch.cuda

    def map_python_to_cpp_type(self, ty: str) -> str:
        if ty.startswith("*"):
            return "CUdeviceptr"
        return {"i1": "int8_t", "i8": "int8_t", "i16": "int16_t", "i32": "int32_t", "i64": "int64_t",
                "u1": "uint8_t", "u8": "uint8_t", "u16": "uint16_t", "u32": "uint32_t", "u64": "uint64_t",
                "fp16": "double", "bf16": "double", "fp32": "double", "f32": "double", "fp64": "double"}[ty]

    def get_benchmarker(self):
        from triton.testing import do_bench

        return do_bench

    def get_empty_cache_for_benchmark(self):
        import torch

        return torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int, device="cuda")

    def clear_cache(self, cache) -> None:
        cache.zero_()
