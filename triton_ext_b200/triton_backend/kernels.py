"""A ready-made K-loop kernel in the shape the LoopSplit extension rewrites, for callers that want a
``@triton.jit`` entry point to the library GEMM (and for bench.py's ``cfg2_jit`` workload).

Importing this module imports Triton's compiler front end; do not import it in a process that runs
Triton's interpreter (TRITON_INTERPRET=1).
"""
import math

import triton
import triton.language as tl


@triton.jit
def dot_kloop(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn,
              K_MAIN, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """C = cast(A @ B), fp32 accumulation. K iterations below K_MAIN load whole tiles; from K_MAIN on the
    loads are masked against K. Rows and columns are masked everywhere, so any M and N work."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    rows = rm[:, None] < M
    cols = rn[None, :] < N
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a_ptrs = a_ptr + rm[:, None] * stride_am + (k + rk)[None, :] * stride_ak
        b_ptrs = b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :] * stride_bn
        if k < K_MAIN:
            a = tl.load(a_ptrs, mask=rows, other=0.0)
            b = tl.load(b_ptrs, mask=cols, other=0.0)
        else:
            a = tl.load(a_ptrs, mask=rows & ((k + rk)[None, :] < K), other=0.0)
            b = tl.load(b_ptrs, mask=((k + rk)[:, None] < K) & cols, other=0.0)
        acc = tl.dot(a, b, acc)
    c_ptrs = c_ptr + rm[:, None] * stride_cm + rn[None, :] * stride_cn
    tl.store(c_ptrs, acc.to(c_ptr.dtype.element_ty), mask=rows & cols)


def launch_dot_kloop(a, b, c, block=(128, 128, 128), k_main=None) -> None:
    """dot_kloop[grid](...) for 2-D tensors a [M, K], b [K, N], c [M, N]; call under triton_backend.activate()."""
    m, k = a.shape
    n = b.shape[1]
    bm, bn, bk = block
    if k_main is None:
        k_main = (k // bk) * bk
    dot_kloop[(math.ceil(m / bm), math.ceil(n / bn))](
        a, b, c, m, n, k, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1), k_main,
        BLOCK_M=bm, BLOCK_N=bn, BLOCK_K=bk)
