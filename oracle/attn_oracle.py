"""CPU restatement of the reference's fused attention forward. TEST INFRASTRUCTURE, not product code: only
tests/, __graft_entry__.smoke() and bench.py's CPU legs may import this file.

  attention_blockwise  the algorithm of `_attn_fwd` / `_attn_fwd_inner`
                       (pass/LoopSplit/06-fused-attention.py:164-240 and :43-90) block by block in numpy fp32:
                       base-2 online softmax, the `start_n >= causal_start` compare LoopSplit splits on (:64),
                       the -1.0e6 additive mask (:66), l_i starting at 1.0 (:222), P rounded to the input type
                       before the second dot (:81-84; e5m2 for fp8 tensors), M = m_i + log2(l_i) (:236).
  attention_eager      the formula the reference's own test compares its kernel with (`test_op`, :697-703):
                       softmax(q k^T * sm_scale with -inf above the diagonal) rounded to the input type, times v.

Pinned by tests/test_attention_oracle.py against outputs of the reference kernel itself (run by Triton's CPU
interpreter, tests/golden/make_attn_golden.py -> tests/golden/attn_golden.npz).
"""
from __future__ import annotations

import numpy as np
import torch


def _round_to(x: np.ndarray, dtype: torch.dtype, interpreter_cast: bool = False) -> np.ndarray:
    """fp32 array rounded to `dtype` (nearest even) and widened back to fp32. With `interpreter_cast` a float8_e5m2
    conversion is done by the Triton interpreter's own routine instead (triton 3.6.0 `_convert_float` in its RTNE
    mode, which is what `x.to(tl.float8e5)` reaches there). That routine rounds half up and ORs a mantissa carry into
    the exponent field instead of adding it, so a value whose mantissa rounds up to 2.0 keeps its exponent when the
    biased exponent is odd (1.9 -> 1.0, not 2.0). It is what produced the fp8 golden vectors, and only pinning the
    restatement against them uses it; a GPU (`cvt.rn.satfinite.e5m2x2.f32`) rounds to nearest even."""
    if interpreter_cast and dtype == torch.float8_e5m2:
        import os
        os.environ["TRITON_INTERPRET"] = "1"  # as oracle/interp_dot.py: must be set before triton is first imported
        import triton.language as tl
        from triton._C.libtriton import ir
        from triton.runtime.interpreter import _convert_float
        x32 = np.ascontiguousarray(x, dtype=np.float32)
        b8 = _convert_float(x32, tl.float32, tl.float8e5, ir.ROUNDING_MODE.RTNE).astype(np.uint8).reshape(x32.shape)
        return torch.from_numpy(b8).view(torch.float8_e5m2).float().numpy()
    return torch.from_numpy(np.ascontiguousarray(x)).to(dtype).float().numpy()


def attention_blockwise(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, sm_scale: float,
                        block_m: int = 128, block_n: int = 128, skip_above_diagonal: bool = False,
                        interpreter_cast: bool = False):
    """Returns (out [Z,H,N,D] in q.dtype, M [Z,H,N] fp32). N must be a multiple of both block sizes, as in
    the reference. With skip_above_diagonal the KV loop of a causal tile stops after the diagonal block
    (the blocks it leaves out contribute p == 0 and alpha == 1 exactly). float8_e5m2 tensors give the reference's
    fp8 forward (P and the output rounded to e5m2); `interpreter_cast` selects the interpreter's own
    conversion for both (see `_round_to`)."""
    z, h, n, d = q.shape
    assert n % block_m == 0 and n % block_n == 0
    dt = q.dtype
    qf, kf, vf = (t.float().numpy() for t in (q, k, v))
    out = np.empty((z, h, n, d), dtype=np.float32)
    m_out = np.empty((z, h, n), dtype=np.float32)
    qk_scale = np.float32(np.float32(sm_scale) * np.float32(1.44269504))
    for iz in range(z):
        for ih in range(h):
            for start_m in range(n // block_m):
                offs_m = start_m * block_m + np.arange(block_m)
                qt = qf[iz, ih, offs_m]
                m_i = np.full(block_m, -np.inf, dtype=np.float32)
                l_i = np.ones(block_m, dtype=np.float32)
                acc = np.zeros((block_m, d), dtype=np.float32)
                causal_start = start_m * block_m if causal else n
                hi = n
                if causal and skip_above_diagonal:
                    hi = min(n, (start_m + 1) * block_m)
                for start_n in range(0, hi, block_n):
                    kt = kf[iz, ih, start_n:start_n + block_n]
                    qk = (qt @ kt.T).astype(np.float32)
                    if start_n >= causal_start:  # the on-band loop after LoopSplit
                        mask = offs_m[:, None] >= (start_n + np.arange(block_n))[None, :]
                        qk = qk * qk_scale + np.where(mask, np.float32(0), np.float32(-1.0e6))
                        m_ij = np.maximum(m_i, qk.max(axis=1))
                        qk = qk - m_ij[:, None]
                    else:                         # the off-band loop
                        m_ij = np.maximum(m_i, qk.max(axis=1) * qk_scale)
                        qk = qk * qk_scale - m_ij[:, None]
                    p = np.exp2(qk.astype(np.float32)).astype(np.float32)
                    l_ij = p.sum(axis=1, dtype=np.float32)
                    alpha = np.exp2(m_i - m_ij).astype(np.float32)
                    l_i = l_i * alpha + l_ij
                    acc = acc * alpha[:, None]
                    acc = acc + _round_to(p, dt, interpreter_cast) @ vf[iz, ih, start_n:start_n + block_n]
                    m_i = m_ij
                m_out[iz, ih, offs_m] = m_i + np.log2(l_i)
                out[iz, ih, offs_m] = acc / l_i[:, None]
    if interpreter_cast and dt == torch.float8_e5m2:
        return torch.from_numpy(_round_to(out, dt, True)).to(dt), torch.from_numpy(m_out)
    return torch.from_numpy(out).to(dt), torch.from_numpy(m_out)


def attention_eager(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, sm_scale: float,
                    round_p: bool = True) -> torch.Tensor:
    """fp32 result of the reference test's formula; works for any N_CTX."""
    n = q.shape[2]
    p = torch.matmul(q.float(), k.float().transpose(2, 3)) * sm_scale
    if causal:
        tril = torch.tril(torch.ones((n, n), dtype=torch.bool))
        p = p.masked_fill(~tril, float("-inf"))
    p = torch.softmax(p, dim=-1)
    if round_p:
        p = p.to(q.dtype).float()
    return torch.matmul(p, v.float())


def logsumexp2(q: torch.Tensor, k: torch.Tensor, causal: bool, sm_scale: float) -> torch.Tensor:
    """What M holds: log2 of the row sums of exp2(scores * sm_scale * log2 e), fp64 arithmetic."""
    n = q.shape[2]
    s = torch.matmul(q.double(), k.double().transpose(2, 3)) * (sm_scale * 1.4426950408889634)
    if causal:
        tril = torch.tril(torch.ones((n, n), dtype=torch.bool))
        s = s.masked_fill(~tril, float("-inf"))
    return (torch.logsumexp(s * 0.6931471805599453, dim=-1) * 1.4426950408889634).float()


def attention_grads_eager(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d_o: torch.Tensor, causal: bool,
                          sm_scale: float):
    """(dq, dk, dv) by autograd through the eager formula in fp32, as the reference's test obtains its reference
    gradients (`ref_out.backward(dout)`, 06-fused-attention.py:704-707), without the rounding of P."""
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    n = q.shape[2]
    p = torch.matmul(qf, kf.transpose(2, 3)) * sm_scale
    if causal:
        tril = torch.tril(torch.ones((n, n), dtype=torch.bool))
        p = p.masked_fill(~tril, float("-inf"))
    out = torch.matmul(torch.softmax(p, dim=-1), vf)
    out.backward(d_o.float())
    return qf.grad, kf.grad, vf.grad

