"""ctypes binding of the fused attention forward (include/b200_attention.h).

Host-side mirror of the reference's `attention(q, k, v, causal, sm_scale)` forward
(pass/LoopSplit/06-fused-attention.py:583-642, `_attention.forward`): same argument order and meaning,
q / k / v of shape [Z, H, N_CTX, HEAD_DIM]; returns the output and, on request, the per-row
`m + log2(l)` vector the reference saves for its backward pass.

torch is used for device memory and streams only. There is no fallback: if the shared library is
missing or no B200 is present the calls raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import backend as B


class AttnProblem(ctypes.Structure):
    _fields_ = [
        ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("n_ctx", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("dtype", ctypes.c_int32), ("causal", ctypes.c_int32),
        ("sm_scale", ctypes.c_float), ("reserved", ctypes.c_int32 * 5),
    ]


_bound = False


def _lib() -> ctypes.CDLL:
    global _bound
    lib = B.load_library()
    if not _bound:
        vp = ctypes.c_void_p
        pp = ctypes.POINTER(AttnProblem)
        lib.tx_attn_fwd.argtypes = [pp, vp, vp, vp, vp, vp, vp]
        lib.tx_attn_fwd.restype = ctypes.c_int
        lib.tx_attn_check.argtypes = [vp]
        lib.tx_attn_check.restype = ctypes.c_int
        lib.tx_attn_fwd_host.argtypes = [pp, vp, vp, vp, vp, vp]
        lib.tx_attn_fwd_host.restype = ctypes.c_int
        lib.tx_attn_bwd.argtypes = [pp] + [vp] * 10
        lib.tx_attn_bwd.restype = ctypes.c_int
        lib.tx_attn_flops.argtypes = [pp]
        lib.tx_attn_flops.restype = ctypes.c_double
        lib.tx_attn_kernel_launches.restype = ctypes.c_uint64
        lib.tx_attn_last_error.restype = ctypes.c_char_p
        _bound = True
    return lib


def _raise(lib, rc: int):
    raise B.DotError(rc, lib.tx_attn_last_error().decode())


def make_problem(z: int, h: int, n_ctx: int, head_dim: int, dtype: torch.dtype, causal: bool,
                 sm_scale: float) -> AttnProblem:
    if dtype not in (torch.float16, torch.bfloat16, torch.float8_e5m2):
        raise B.DotError(B.TXD_ERR_UNSUPPORTED, f"attention dtype {dtype}: f16, bf16 and (forward only) float8_e5m2 are built")
    return AttnProblem(batch=z, heads=h, n_ctx=n_ctx, head_dim=head_dim, dtype=B._DTYPES[dtype],
                       causal=1 if causal else 0, sm_scale=float(sm_scale))


def kv_loop_split(n_ctx: int, q_start: int, causal: bool, block: int = 128) -> tuple[int, int]:
    """(blocks visited, blocks of them that run unmasked) for the 128 query rows starting at `q_start`: the
    arithmetic the kernel uses per sub-tile. It is LoopSplit applied to the reference's KV loop
    (`for start_n in range(0, hi, BLOCK_N): if start_n >= causal_start`, 06-fused-attention.py:59-64): the
    off-band loop is [0, unmasked * block), the on-band loop the rest."""
    if q_start >= n_ctx:
        return 0, 0
    all_blocks = -(-n_ctx // block)
    n = min(all_blocks, q_start // block + 1) if causal else all_blocks
    last_masked = n > 0 and (causal or (n_ctx % block != 0 and n == all_blocks))
    return n, n - 1 if last_masked else n


def fp8_v_layout(v: torch.Tensor) -> torch.Tensor:
    """V as the fp8 forward takes it: shape [Z, H, N_CTX, HEAD_DIM] with the N_CTX index contiguous in memory
    ([Z, H, HEAD_DIM, N_CTX] storage), which is how the reference lays V out for float8_e5m2
    (`v.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)`, 06-fused-attention.py:777-778); the fp8 second dot
    takes its B operand K-major. Returns `v` itself when it already is, else a copy."""
    z, h, n, d = v.shape
    if v.stride() == (h * n * d, n * d, 1, n):
        return v
    return v.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)


def _operands(q, k, v):
    """Contiguous q, k and v in the layout the kernels read (fp8: V with N_CTX contiguous)."""
    q, k = q.contiguous(), k.contiguous()
    v = fp8_v_layout(v) if v.dtype == torch.float8_e5m2 else v.contiguous()
    return q, k, v


def flops(problem: AttnProblem) -> float:
    return float(_lib().tx_attn_flops(ctypes.byref(problem)))


def kernel_launches() -> int:
    return int(_lib().tx_attn_kernel_launches())


def attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, sm_scale: float, *,
                      out: Optional[torch.Tensor] = None, return_m: bool = False, check: bool = False):
    """softmax(q k^T * sm_scale [+ causal mask]) v on the current CUDA stream (asynchronous unless `check`).
    With float8_e5m2 tensors this is the reference's fp8 forward (:81-82, :191): P is rounded to e5m2 before the second
    dot, the output is e5m2, and V is read with N_CTX contiguous (`fp8_v_layout`; any other V is copied into it)."""
    lib = _lib()
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise B.DotError(B.TXD_ERR_NO_DEVICE, "attention_forward takes CUDA tensors; use attention_forward_host for host tensors")
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape or not (q.dtype == k.dtype == v.dtype):
        raise B.DotError(B.TXD_ERR_INVALID, "q, k, v must be [Z, H, N_CTX, HEAD_DIM] tensors of one shape and type")
    q, k, v = _operands(q, k, v)
    z, h, n, d = q.shape
    pr = make_problem(z, h, n, d, q.dtype, causal, sm_scale)
    if out is None:
        out = torch.empty_like(q)
    m = torch.empty((z, h, n), dtype=torch.float32, device=q.device) if return_m else None
    stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    with torch.cuda.device(q.device):
        rc = lib.tx_attn_fwd(ctypes.byref(pr), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                             m.data_ptr() if m is not None else None, stream)
        if rc:
            _raise(lib, rc)
        if check:
            rc = lib.tx_attn_check(stream)
            if rc:
                _raise(lib, rc)
    return (out, m) if return_m else out


def check(device=None) -> None:
    """Synchronise the current stream and raise if a bounded wait ran out inside the kernel."""
    lib = _lib()
    dev = device if device is not None else torch.cuda.current_device()
    with torch.cuda.device(dev):
        rc = lib.tx_attn_check(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc:
        _raise(lib, rc)


def attention_forward_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, sm_scale: float, *,
                           out: Optional[torch.Tensor] = None, m: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same through host tensors (pinned or pageable): H2D copies, kernel, D2H copy, synchronise."""
    lib = _lib()
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise B.DotError(B.TXD_ERR_INVALID, "attention_forward_host takes host tensors")
    q, k, v = _operands(q, k, v)
    z, h, n, d = q.shape
    pr = make_problem(z, h, n, d, q.dtype, causal, sm_scale)
    if out is None:
        out = torch.empty_like(q)
    rc = lib.tx_attn_fwd_host(ctypes.byref(pr), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                              m.data_ptr() if m is not None else None)
    if rc:
        _raise(lib, rc)
    return out


def attention_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, m: torch.Tensor,
                       d_o: torch.Tensor, causal: bool, sm_scale: float, *, check: bool = False):
    """(dq, dk, dv) of attention_forward, from its output `o`, its row vector `m` and the output gradient `d_o`
    (reference `_attention.backward`, 06-fused-attention.py:645-688)."""
    lib = _lib()
    tensors = [t.contiguous() for t in (q, k, v, o, d_o)]
    if not all(t.is_cuda for t in tensors) or not m.is_cuda:
        raise B.DotError(B.TXD_ERR_NO_DEVICE, "attention_backward takes CUDA tensors")
    q, k, v, o, d_o = tensors
    if not (q.shape == k.shape == v.shape == o.shape == d_o.shape) or not (q.dtype == k.dtype == v.dtype == o.dtype == d_o.dtype):
        raise B.DotError(B.TXD_ERR_INVALID, "q, k, v, o, d_o must share shape and type")
    z, h, n, d = q.shape
    m = m.contiguous().float()
    pr = make_problem(z, h, n, d, q.dtype, causal, sm_scale)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    with torch.cuda.device(q.device):
        rc = lib.tx_attn_bwd(ctypes.byref(pr), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(),
                             m.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), stream)
        if rc:
            _raise(lib, rc)
        if check:
            rc = lib.tx_attn_check(stream)
            if rc:
                _raise(lib, rc)
    return dq, dk, dv


class _Attention(torch.autograd.Function):
    """The reference's `_attention` autograd function (06-fused-attention.py:581-688) on this library's kernels."""

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale):
        o, m = attention_forward(q, k, v, causal, sm_scale, return_m=True)
        ctx.save_for_backward(q, k, v, o, m)
        ctx.causal, ctx.sm_scale = causal, sm_scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, m = ctx.saved_tensors
        dq, dk, dv = attention_backward(q, k, v, o, m, d_o, ctx.causal, ctx.sm_scale)
        return dq, dk, dv, None, None


attention = _Attention.apply

