"""TEST INFRASTRUCTURE — not part of the product path.

The numeric oracle: one `tt.dot` K-loop GEMM written as a Triton kernel and executed on the host by
Triton's interpreter (``TRITON_INTERPRET=1``; triton 3.6.0, a third-party wheel — the reference pins
no Triton version, its CI builds Triton's main branch, ci/fetch-triton-hash.py:11-13).

What it restates from the reference: the shape of the loop its LoopSplit pass targets and the
tl.dot / epilogue idioms of its only kernels —
  * K loop with a compare of the induction variable against a loop-invariant bound, one branch per
    side (pass/LoopSplit/06-fused-attention.py:59-89, compare at :64); here the compare is
    ``k < K_MAIN`` and the branches are the unmasked and the masked operand loads;
  * ``acc = tl.dot(a, b, acc)`` into an fp32 accumulator (:85, accumulator created at :222);
  * scale then cast epilogue (:236-240): ``acc * alpha * row_scale[:, None] * col_scale[None, :]``.

Two facts about the 3.6.0 interpreter shape this file:
  * bf16 tensors are held as uint16 bit patterns and `tl.dot` multiplies those integers, so bf16
    operands are widened to fp32 inside the kernel before the dot (exact: bf16 is a subset of fp32);
  * the interpreter's fp32->bf16 cast truncates, the GPU rounds to nearest even; results are compared
    with a tolerance, never bit for bit.

The interpreter runs programs one after another in Python, so `tile_ids` can restrict a run to a
sample of output tiles; the rest of C is left untouched.
"""
from __future__ import annotations

import os

os.environ["TRITON_INTERPRET"] = "1"  # must be set before triton is imported

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402


@triton.jit
def _dot_kloop_kernel(a_ptr, b_ptr, c_ptr, rs_ptr, cs_ptr, tile_ptr,
                      M, N, K, K_MAIN,
                      stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn,
                      alpha, TILES_N,
                      BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr,
                      WIDEN: tl.constexpr, HAS_RS: tl.constexpr, HAS_CS: tl.constexpr):
    tile = tl.load(tile_ptr + tl.program_id(0))
    pid_m = tile // TILES_N
    pid_n = tile % TILES_N
    offs_m = pid_m * BLOCK_M + tl.arange(0, BLOCK_M)
    offs_n = pid_n * BLOCK_N + tl.arange(0, BLOCK_N)
    offs_k = tl.arange(0, BLOCK_K)
    m_ok = offs_m < M
    n_ok = offs_n < N
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a_ptrs = a_ptr + offs_m[:, None] * stride_am + (k + offs_k)[None, :] * stride_ak
        b_ptrs = b_ptr + (k + offs_k)[:, None] * stride_bk + offs_n[None, :] * stride_bn
        if k < K_MAIN:
            # main loop: the whole K block lies inside [0, K)
            a = tl.load(a_ptrs, mask=m_ok[:, None], other=0.0)
            b = tl.load(b_ptrs, mask=n_ok[None, :], other=0.0)
        else:
            # remainder: mask the columns / rows past K
            k_ok = (k + offs_k) < K
            a = tl.load(a_ptrs, mask=m_ok[:, None] & k_ok[None, :], other=0.0)
            b = tl.load(b_ptrs, mask=k_ok[:, None] & n_ok[None, :], other=0.0)
        if WIDEN:
            a = a.to(tl.float32)
            b = b.to(tl.float32)
        acc = tl.dot(a, b, acc)
    acc = acc * alpha
    if HAS_RS:
        rs = tl.load(rs_ptr + offs_m, mask=m_ok, other=1.0)
        acc = acc * rs[:, None]
    if HAS_CS:
        cs = tl.load(cs_ptr + offs_n, mask=n_ok, other=1.0)
        acc = acc * cs[None, :]
    c_ptrs = c_ptr + offs_m[:, None] * stride_cm + offs_n[None, :] * stride_cn
    tl.store(c_ptrs, acc.to(c_ptr.dtype.element_ty), mask=m_ok[:, None] & n_ok[None, :])


def interp_dot(a: torch.Tensor, b: torch.Tensor, *, out_dtype: torch.dtype, block_m: int = 64,
               block_n: int = 64, block_k: int = 32, row_scale: torch.Tensor | None = None,
               col_scale: torch.Tensor | None = None, alpha: float = 1.0,
               tile_ids=None, out: torch.Tensor | None = None, k_main: int | None = None) -> torch.Tensor:
    """Run the oracle kernel on CPU tensors. `a` is [M, K], `b` is [K, N] (any strides).

    `k_main` is the LoopSplit mid point (default: floor(K / BLOCK_K) * BLOCK_K); any value in
    [0, that default] gives the same numbers because the remainder branch only adds masking.
    """
    assert not a.is_cuda and not b.is_cuda, "the oracle runs on the host"
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    tiles_m, tiles_n = triton.cdiv(m, block_m), triton.cdiv(n, block_n)
    if out is None:
        out = torch.zeros((m, n), dtype=out_dtype)
    if m == 0 or n == 0:
        return out
    if tile_ids is None:
        tile_ids = np.arange(tiles_m * tiles_n, dtype=np.int32)
    tiles = torch.as_tensor(np.asarray(tile_ids, dtype=np.int32))
    if tiles.numel() == 0:
        return out
    if k_main is None:
        k_main = (k // block_k) * block_k
    widen = a.dtype == torch.bfloat16
    dummy = torch.zeros(1, dtype=torch.float32)
    _dot_kloop_kernel[(tiles.numel(),)](
        a, b, out, row_scale if row_scale is not None else dummy, col_scale if col_scale is not None else dummy,
        tiles, m, n, k, k_main,
        a.stride(0), a.stride(1), b.stride(0), b.stride(1), out.stride(0), out.stride(1),
        float(alpha), tiles_n,
        BLOCK_M=block_m, BLOCK_N=block_n, BLOCK_K=block_k,
        WIDEN=widen, HAS_RS=row_scale is not None, HAS_CS=col_scale is not None)
    return out


def tile_mask(m: int, n: int, block_m: int, block_n: int, tile_ids) -> torch.Tensor:
    """Boolean [m, n] mask of the elements covered by `tile_ids`."""
    tiles_n = (n + block_n - 1) // block_n
    mask = torch.zeros((m, n), dtype=torch.bool)
    for t in np.asarray(tile_ids).tolist():
        tm, tn = divmod(int(t), tiles_n)
        mask[tm * block_m:(tm + 1) * block_m, tn * block_n:(tn + 1) * block_n] = True
    return mask


def sample_tiles(m: int, n: int, block_m: int, block_n: int, count: int, seed: int) -> np.ndarray:
    """A seeded sample of output tiles that always holds the four corner tiles (edge tiles included)."""
    tiles_m, tiles_n = (m + block_m - 1) // block_m, (n + block_n - 1) // block_n
    total = tiles_m * tiles_n
    corners = {0, tiles_n - 1, (tiles_m - 1) * tiles_n, total - 1}
    rng = np.random.default_rng(seed)
    extra = rng.choice(total, size=min(count, total), replace=False).tolist()
    ids = sorted(corners | set(int(x) for x in extra))
    return np.asarray(ids[:max(count, len(corners))] if len(ids) > count + len(corners) else ids, dtype=np.int32)
