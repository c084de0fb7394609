"""ctypes binding of the `b200_dot` backend extension (include/b200_dot.h).

This is the host-side mirror of what a `tl.dot` call means in the reference's only kernels
(pass/LoopSplit/06-fused-attention.py:63,85 — `tl.dot(a, b)` / `tl.dot(a, b, acc)` with an fp32
accumulator, followed by the scale and cast idioms of :66,78,237,240): one call computes
``cast(alpha * row_scale[:, None] * col_scale[None, :] * (A @ B))`` with fp32 accumulation.

torch is used for device memory and streams only. There is no fallback: if the shared library is
missing or no B200 is present the calls raise.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch

_LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
_LIB_PATH = os.path.join(_LIB_DIR, "libb200_dot.so")

TXD_OK = 0
TXD_ERR_INVALID = 1
TXD_ERR_UNSUPPORTED = 2
TXD_ERR_CUDA = 3
TXD_ERR_DEVICE_TIMEOUT = 4
TXD_ERR_NO_DEVICE = 5

TXD_F16, TXD_BF16, TXD_F8E4M3, TXD_F32, TXD_F8E5M2 = 0, 1, 2, 3, 4
TXD_ROW_MAJOR, TXD_COL_MAJOR = 0, 1
TXD_SCHED_AUTO, TXD_SCHED_DATA_PARALLEL, TXD_SCHED_STREAM_K, TXD_SCHED_HYBRID = 0, 1, 2, 3

_DTYPES = {
    torch.float16: TXD_F16,
    torch.bfloat16: TXD_BF16,
    torch.float8_e4m3fn: TXD_F8E4M3,
    torch.float32: TXD_F32,
    torch.float8_e5m2: TXD_F8E5M2,
}


class DotError(RuntimeError):
    """A b200_dot entry point returned a non-zero tx_dot_status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"b200_dot status {status}: {message}")
        self.status = status


class Problem(ctypes.Structure):
    _fields_ = [
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32),
        ("ab_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("a_layout", ctypes.c_int32), ("b_layout", ctypes.c_int32),
        ("has_row_scale", ctypes.c_int32), ("has_col_scale", ctypes.c_int32),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
        ("alpha", ctypes.c_float),
    ]


class Config(ctypes.Structure):
    _fields_ = [
        ("block_n", ctypes.c_int32), ("stages", ctypes.c_int32), ("swap_ab", ctypes.c_int32),
        ("schedule", ctypes.c_int32), ("group_m", ctypes.c_int32), ("max_ctas", ctypes.c_int32),
        ("k_split_point", ctypes.c_int32), ("cta_pair", ctypes.c_int32),
        ("atoms", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class PlanInfo(ctypes.Structure):
    _fields_ = [
        ("block_m", ctypes.c_int32), ("block_n", ctypes.c_int32), ("block_k", ctypes.c_int32),
        ("stages", ctypes.c_int32), ("swap_ab", ctypes.c_int32), ("schedule", ctypes.c_int32),
        ("group_m", ctypes.c_int32), ("grid", ctypes.c_int32),
        ("k_main_iters", ctypes.c_int32), ("k_tail_iters", ctypes.c_int32),
        ("k_tail_mmas", ctypes.c_int32), ("smem_bytes", ctypes.c_int32),
        ("tmem_columns", ctypes.c_int32), ("cta_pair", ctypes.c_int32),
        ("scratch_bytes", ctypes.c_int64), ("flops", ctypes.c_double),
        ("algorithmic_bytes", ctypes.c_double),
    ]

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_ if name != "reserved"}


_lib = None


def load_library() -> ctypes.CDLL:
    """dlopen libb200_dot.so from the package's lib/ directory (built by __graft_entry__.build())."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} is missing: build the CUDA extension first "
            "(python -c 'import __graft_entry__ as g; g.build()'); there is no CPU fallback")
    lib = ctypes.CDLL(_LIB_PATH)
    vp, i32, f32p = ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p
    lib.tx_dot_device_count.restype = ctypes.c_int
    lib.tx_dot_last_error.restype = ctypes.c_char_p
    lib.tx_dot_kernel_launches.restype = ctypes.c_uint64
    lib.tx_dot_plan_create.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Config), ctypes.POINTER(vp)]
    lib.tx_dot_plan_preview.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Config), i32, ctypes.POINTER(PlanInfo)]
    lib.tx_dot_plan_query.argtypes = [vp, ctypes.POINTER(PlanInfo)]
    lib.tx_dot_run.argtypes = [vp, vp, vp, vp, f32p, f32p, vp]
    lib.tx_dot_plan_check.argtypes = [vp, vp]
    lib.tx_dot_run_host.argtypes = [vp, vp, vp, vp, f32p, f32p]
    lib.tx_dot_plan_destroy.argtypes = [vp]
    lib.tx_dot_run_to_slots.argtypes = [vp, vp, vp, ctypes.POINTER(vp), i32, i32, vp]
    lib.tx_dot_reduce_slots.argtypes = [vp, i32, i32, i32, i32, vp, i32, ctypes.c_int64, f32p, f32p, ctypes.c_float, vp]
    lib.tx_dot_run_to_slots_part.argtypes = [vp, vp, vp, ctypes.POINTER(vp), i32, i32, i32, i32, vp]
    lib.tx_dot_reduce_slots_part.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, i32, ctypes.c_int64, f32p, f32p,
                                             ctypes.c_float, vp]
    for name in ("tx_dot_plan_create", "tx_dot_plan_preview", "tx_dot_plan_query", "tx_dot_run",
                 "tx_dot_plan_check", "tx_dot_run_host", "tx_dot_plan_destroy", "tx_dot_run_to_slots",
                 "tx_dot_reduce_slots", "tx_dot_run_to_slots_part", "tx_dot_reduce_slots_part"):
        getattr(lib, name).restype = ctypes.c_int
    _lib = lib
    return lib


def _check(rc: int) -> None:
    if rc != TXD_OK:
        raise DotError(rc, load_library().tx_dot_last_error().decode())


def kernel_launches() -> int:
    return int(load_library().tx_dot_kernel_launches())


def _layout_and_ld(t: torch.Tensor, name: str) -> tuple[int, int]:
    """(layout, leading dimension) of a 2-D tensor addressed as [rows, cols]."""
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D")
    rows, cols = t.shape
    s0, s1 = t.stride()
    if s1 == 1 or cols == 1:
        return TXD_ROW_MAJOR, max(s0 if rows > 1 else cols, cols, 1)
    if s0 == 1 or rows == 1:
        return TXD_COL_MAJOR, max(s1 if cols > 1 else rows, rows, 1)
    raise ValueError(f"{name} must have a unit stride in one dimension (strides {t.stride()})")


def make_problem(m: int, n: int, k: int, ab_dtype: torch.dtype, out_dtype: torch.dtype, *,
                 a_layout: int = TXD_ROW_MAJOR, b_layout: int = TXD_ROW_MAJOR,
                 lda: Optional[int] = None, ldb: Optional[int] = None, ldc: Optional[int] = None,
                 row_scale: bool = False, col_scale: bool = False, alpha: float = 1.0) -> Problem:
    pr = Problem()
    pr.m, pr.n, pr.k = m, n, k
    pr.ab_dtype, pr.out_dtype = _DTYPES[ab_dtype], _DTYPES[out_dtype]
    pr.a_layout, pr.b_layout = a_layout, b_layout
    pr.lda = lda if lda is not None else (k if a_layout == TXD_ROW_MAJOR else m)
    pr.ldb = ldb if ldb is not None else (n if b_layout == TXD_ROW_MAJOR else k)
    pr.ldc = ldc if ldc is not None else n
    pr.has_row_scale, pr.has_col_scale = int(row_scale), int(col_scale)
    pr.alpha = alpha
    return pr


def make_config(**kw) -> Config:
    cfg = Config()
    for key, val in kw.items():
        if not hasattr(cfg, key):
            raise TypeError(f"unknown tx_dot_config field {key!r}")
        setattr(cfg, key, int(val))
    return cfg


def preview(problem: Problem, config: Optional[Config] = None, sm_count: int = 148) -> dict:
    """Tile-selection result for a problem without touching a GPU."""
    info = PlanInfo()
    _check(load_library().tx_dot_plan_preview(ctypes.byref(problem), ctypes.byref(config) if config else None,
                                              sm_count, ctypes.byref(info)))
    return info.as_dict()


def _check_scale(t: Optional[torch.Tensor], length: int, device: torch.device, name: str) -> None:
    """A scale vector is read by the kernel as `length` consecutive floats: anything else is refused here,
    before a launch could read past it."""
    if t is None:
        return
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32, got {t.dtype}")
    if t.dim() != 1 or t.numel() != length or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous vector of {length} elements, got shape {tuple(t.shape)} "
                         f"strides {t.stride()}")
    if not t.is_cuda or t.device != device:
        raise ValueError(f"{name} must be a CUDA tensor on {device}, got {t.device}")


def _span_elements(t: torch.Tensor) -> int:
    """Elements between the first and one past the last element a strided 2-D tensor addresses."""
    if t.numel() == 0:
        return 0
    return 1 + sum((n - 1) * abs(st) for n, st in zip(t.shape, t.stride()))


class DotPlan:
    """Owns one tx_dot_plan. Create once per (shape, dtype, layout); run many times.
    One plan serves one host thread at a time (it caches tensor maps keyed by the last pointers)."""

    def __init__(self, problem: Problem, config: Optional[Config] = None):
        lib = load_library()
        self._lib = lib
        self.problem = problem
        handle = ctypes.c_void_p()
        _check(lib.tx_dot_plan_create(ctypes.byref(problem), ctypes.byref(config) if config else None,
                                      ctypes.byref(handle)))
        self._h = handle
        info = PlanInfo()
        _check(lib.tx_dot_plan_query(self._h, ctypes.byref(info)))
        self.info = info.as_dict()

    def run(self, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
            row_scale: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None,
            stream: Optional[torch.cuda.Stream] = None) -> None:
        s = stream if stream is not None else torch.cuda.current_stream(c.device)
        self._check_buffers(a, b, c, row_scale, col_scale)
        _check(self._lib.tx_dot_run(
            self._h, a.data_ptr(), b.data_ptr(), c.data_ptr(),
            row_scale.data_ptr() if row_scale is not None else None,
            col_scale.data_ptr() if col_scale is not None else None,
            ctypes.c_void_p(s.cuda_stream)))

    def _check_buffers(self, a, b, c, row_scale, col_scale) -> None:
        """The buffers must hold what the plan's problem says the kernel will read and write."""
        pr = self.problem
        dev = c.device
        if not (a.is_cuda and b.is_cuda and c.is_cuda) or a.device != dev or b.device != dev:
            raise ValueError(f"a, b and c must be CUDA tensors on one device (got {a.device}, {b.device}, {c.device})")
        if _DTYPES.get(a.dtype) != pr.ab_dtype or _DTYPES.get(b.dtype) != pr.ab_dtype:
            raise TypeError(f"operand dtypes {a.dtype}, {b.dtype} do not match the plan")
        if _DTYPES.get(c.dtype) != pr.out_dtype:
            raise TypeError(f"output dtype {c.dtype} does not match the plan's")
        if pr.m == 0 or pr.n == 0:
            return
        a_need = ((pr.m - 1) * pr.lda + pr.k) if pr.a_layout == TXD_ROW_MAJOR else ((pr.k - 1) * pr.lda + pr.m)
        b_need = ((pr.k - 1) * pr.ldb + pr.n) if pr.b_layout == TXD_ROW_MAJOR else ((pr.n - 1) * pr.ldb + pr.k)
        c_need = (pr.m - 1) * pr.ldc + pr.n
        if pr.k > 0 and (_span_elements(a) < a_need or _span_elements(b) < b_need):
            raise ValueError(f"operand buffers are smaller than the plan's {pr.m}x{pr.n}x{pr.k} problem needs")
        if _span_elements(c) < c_need:
            raise ValueError(f"output buffer addresses {_span_elements(c)} elements, the plan writes {c_need}")
        if (pr.has_row_scale != 0) != (row_scale is not None) or (pr.has_col_scale != 0) != (col_scale is not None):
            raise ValueError("scale vectors must be given exactly when the plan was created with them")
        _check_scale(row_scale, pr.m, dev, "row_scale")
        _check_scale(col_scale, pr.n, dev, "col_scale")

    def run_to_slots(self, a: torch.Tensor, b: torch.Tensor, slot_ptrs: list, rank: int,
                     stream: Optional[torch.cuda.Stream] = None, part: int = 0, parts: int = 1) -> None:
        """K-sharded form: store every tile into slot `rank` of the buffer of the rank owning its rows.
        `slot_ptrs[o]` is the device address of rank o's [world, m/world, n] slot buffer (peer-mapped).
        With parts > 1 only piece `part` of the tile rows is computed: rows [part, part + 1) * (m/world/parts) of
        every owner's slot."""
        s = stream if stream is not None else torch.cuda.current_stream(a.device)
        world = len(slot_ptrs)
        arr = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(p)) for p in slot_ptrs])
        _check(self._lib.tx_dot_run_to_slots_part(self._h, a.data_ptr(), b.data_ptr(), arr, world, rank, part, parts,
                                                  ctypes.c_void_p(s.cuda_stream)))

    def check(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        s = stream if stream is not None else torch.cuda.current_stream()
        _check(self._lib.tx_dot_plan_check(self._h, ctypes.c_void_p(s.cuda_stream)))

    def run_host(self, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor,
                 row_scale: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None) -> None:
        """Host buffers in, host buffer out (copies inside); synchronous."""
        for t in (a, b, c, row_scale, col_scale):
            if t is not None and t.is_cuda:
                raise ValueError("run_host takes CPU tensors")
        _check(self._lib.tx_dot_run_host(
            self._h, a.data_ptr(), b.data_ptr(), c.data_ptr(),
            row_scale.data_ptr() if row_scale is not None else None,
            col_scale.data_ptr() if col_scale is not None else None))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.tx_dot_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def reduce_slots(slots: torch.Tensor, out: torch.Tensor, *, row_scale: Optional[torch.Tensor] = None,
                 col_scale: Optional[torch.Tensor] = None, alpha: float = 1.0,
                 stream: Optional[torch.cuda.Stream] = None, row0: int = 0, rows: Optional[int] = None) -> torch.Tensor:
    """out[r, c] = cast(alpha * rs[r] * cs[c] * sum_s slots[s, r, c]); slots is [world, rows, n], f32 or bf16.
    `row0`, `rows` restrict the call to rows [row0, row0 + rows) of every slot and of `out` (one piece of the exchange)."""
    world, rows_per_rank, n = slots.shape
    if not slots.is_contiguous() or out.stride(1) != 1:
        raise ValueError("slots must be contiguous and out row-major")
    if tuple(out.shape) != (rows_per_rank, n):
        raise ValueError(f"out has shape {tuple(out.shape)}, a slot is {(rows_per_rank, n)}")
    if row_scale is not None and (row_scale.dtype != torch.float32 or row_scale.numel() != rows_per_rank or not row_scale.is_contiguous()):
        raise ValueError(f"row_scale must be {rows_per_rank} contiguous float32 values")
    if col_scale is not None and (col_scale.dtype != torch.float32 or col_scale.numel() != n or not col_scale.is_contiguous()):
        raise ValueError(f"col_scale must be {n} contiguous float32 values")
    if rows is None:
        rows = rows_per_rank - row0
    s = stream if stream is not None else torch.cuda.current_stream(slots.device)
    _check(load_library().tx_dot_reduce_slots_part(
        slots.data_ptr(), world, rows_per_rank, row0, rows, n, _DTYPES[slots.dtype], out.data_ptr(), _DTYPES[out.dtype],
        out.stride(0), row_scale.data_ptr() if row_scale is not None else None,
        col_scale.data_ptr() if col_scale is not None else None, ctypes.c_float(alpha), ctypes.c_void_p(s.cuda_stream)))
    return out


_plan_cache: dict = {}


def dot(a: torch.Tensor, b: torch.Tensor, *, out: Optional[torch.Tensor] = None,
        out_dtype: Optional[torch.dtype] = None, row_scale: Optional[torch.Tensor] = None,
        col_scale: Optional[torch.Tensor] = None, alpha: float = 1.0,
        config: Optional[Config] = None, check: bool = False) -> torch.Tensor:
    """C = cast(alpha * row_scale[:,None] * col_scale[None,:] * (A @ B)), fp32 accumulate, on the GPU.

    `a` is [M, K], `b` is [K, N]; either may be a transposed view (unit stride in one dimension).
    Default output dtype: the operand dtype for f16/bf16, bf16 for fp8 operands.
    """
    if a.dtype != b.dtype:
        raise TypeError(f"tt.dot operands must share a dtype, got {a.dtype} and {b.dtype}")
    m, k = a.shape
    k2, n = b.shape
    if k != k2:
        raise ValueError(f"shape mismatch: A is {tuple(a.shape)}, B is {tuple(b.shape)}")
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else (a.dtype if a.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16)
    # A caller's buffer is written as m x n elements of out_dtype, and a scale vector is read as m (n) floats:
    # anything that is not exactly that is refused here, before any launch.
    if out is not None:
        if tuple(out.shape) != (m, n):
            raise ValueError(f"out has shape {tuple(out.shape)}, the product is {(m, n)}")
        if out.dtype != out_dtype:
            raise TypeError(f"out is {out.dtype} but out_dtype is {out_dtype}")
        if out.stride(1) != 1 and n > 1:
            raise ValueError("out must be row-major")
    for t, length, name in ((row_scale, m, "row_scale"), (col_scale, n, "col_scale")):
        if t is not None and (t.dtype != torch.float32 or t.dim() != 1 or t.numel() != length or not t.is_contiguous()):
            _check_scale(t, length, a.device, name)  # raises with the reason
    if not (a.is_cuda and b.is_cuda):
        raise ValueError("dot() takes CUDA tensors; there is no CPU path")
    if a.device != b.device:
        raise ValueError(f"a is on {a.device}, b on {b.device}")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    elif not out.is_cuda or out.device != a.device:
        raise ValueError(f"out is on {out.device}, the operands on {a.device}")
    _check_scale(row_scale, m, a.device, "row_scale")
    _check_scale(col_scale, n, a.device, "col_scale")
    a_layout, lda = _layout_and_ld(a, "a")
    b_layout, ldb = _layout_and_ld(b, "b")
    ldc = max(out.stride(0), n) if m > 1 else n
    key = (m, n, k, a.dtype, out_dtype, a_layout, b_layout, lda, ldb, ldc, row_scale is not None,
           col_scale is not None, float(alpha), bytes(config) if config is not None else None, a.device.index)
    plan = _plan_cache.get(key)
    if plan is None:
        with torch.cuda.device(a.device):
            pr = make_problem(m, n, k, a.dtype, out_dtype, a_layout=a_layout, b_layout=b_layout, lda=lda, ldb=ldb,
                              ldc=ldc, row_scale=row_scale is not None, col_scale=col_scale is not None, alpha=alpha)
            plan = DotPlan(pr, config)
        _plan_cache[key] = plan
    with torch.cuda.device(a.device):
        plan.run(a, b, out, row_scale, col_scale)
        if check:
            plan.check()
    return out
