"""Seeded inputs for every parity case: the five BASELINE configurations and their scaled-down
siblings. Inputs are always drawn on the CPU from torch.Generator(seed) in fp32 and then cast, so the
oracle and the GPU kernels see bit-identical operands."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class Case:
    name: str
    m: int
    n: int
    k: int
    ab_dtype: torch.dtype
    out_dtype: torch.dtype
    seed: int
    dist: str = "normal"          # "normal" | "uniform" (U[-1,1]) | "mlp" (A ~ N(0,1), B ~ N(0,0.02))
    scales: bool = False          # per-row scale on A, per-column scale on B, both U[0.5, 2]
    block: tuple = (64, 64, 32)   # BLOCK_M, BLOCK_N, BLOCK_K of the oracle program
    a_t: bool = False             # A stored column-major
    b_t: bool = False             # B stored as [N, K] (K contiguous)
    alpha: float = 1.0
    rtol: float = 1e-2
    atol: float = 1e-2


def make_inputs(c: Case):
    """Returns (a [M,K], b [K,N], row_scale or None, col_scale or None) as CPU tensors."""
    g = torch.Generator().manual_seed(c.seed)

    def draw(rows, cols, std=1.0):
        if c.dist == "uniform":
            return torch.rand(rows, cols, generator=g) * 2 - 1
        return torch.randn(rows, cols, generator=g) * std

    a32 = draw(c.m, c.k)
    b32 = draw(c.k, c.n, 0.02 if c.dist == "mlp" else 1.0)
    a = a32.to(c.ab_dtype)
    b = b32.to(c.ab_dtype)
    if c.a_t:
        a = a.t().contiguous().t()
    if c.b_t:
        b = b.t().contiguous().t()
    rs = cs = None
    if c.scales:
        rs = torch.rand(c.m, generator=g) * 1.5 + 0.5
        cs = torch.rand(c.n, generator=g) * 1.5 + 0.5
    return a, b, rs, cs


def reference_fp64(c: Case, a, b, rs, cs) -> torch.Tensor:
    """Exact-arithmetic answer (fp64) for judging both the oracle and the kernels."""
    r = a.double() @ b.double() * c.alpha
    if rs is not None:
        r = r * rs.double()[:, None]
    if cs is not None:
        r = r * cs.double()[None, :]
    return r


f16, bf16, f8, f32 = torch.float16, torch.bfloat16, torch.float8_e4m3fn, torch.float32

# ---- the BASELINE configurations at full size (GPU only; the oracle runs on a tile sample) ----------------
CFG1 = Case("cfg1_fp16_512", 512, 512, 512, f16, f16, seed=0, block=(64, 64, 32))
CFG2 = Case("cfg2_bf16_tail_4096x4096x4160", 4096, 4096, 4160, bf16, bf16, seed=1, dist="uniform", block=(128, 128, 128))
CFG3 = Case("cfg3_bf16_decode_16x4096x14336", 16, 14336, 4096, bf16, bf16, seed=2, dist="mlp", block=(16, 128, 128))
CFG4 = Case("cfg4_fp8_8192_scaled", 8192, 8192, 8192, f8, bf16, seed=3, scales=True, block=(128, 128, 128),
            rtol=3e-2, atol=3e-2)
CFG5 = Case("cfg5_bf16_16384x28672x8192", 16384, 28672, 8192, bf16, bf16, seed=4, dist="mlp", block=(128, 128, 128))

# ---- small cases: oracle-complete in seconds; their oracle outputs are committed under tests/golden/ --------
GOLDEN_CASES = [
    CFG1,
    Case("tail_bf16_256x192x520", 256, 192, 520, bf16, bf16, seed=1, dist="uniform", block=(128, 64, 128)),
    Case("decode_bf16_16x1024x512", 16, 1024, 512, bf16, bf16, seed=2, dist="mlp", block=(16, 128, 128)),
    Case("fp8_scaled_256x256x256", 256, 256, 256, f8, bf16, seed=3, scales=True, block=(64, 64, 128), rtol=3e-2, atol=3e-2),
    Case("ragged_bf16_200x136x72", 200, 136, 72, bf16, bf16, seed=5, block=(64, 64, 32)),
    Case("ragged_f16_f32out_130x72x40", 130, 72, 40, f16, f32, seed=6, block=(64, 64, 32)),
    Case("colmajor_a_bf16_128x128x192", 128, 128, 192, bf16, bf16, seed=7, a_t=True, block=(64, 64, 64)),
    Case("kmajor_b_f16_192x128x128", 192, 128, 128, f16, f16, seed=8, b_t=True, block=(64, 64, 64)),
    Case("alpha_bf16_128x256x64", 128, 256, 64, bf16, bf16, seed=9, alpha=0.125, block=(64, 64, 64)),
    Case("fp8_e4m3_kmajor_128x128x384", 128, 128, 384, f8, bf16, seed=10, b_t=True, scales=True, block=(64, 64, 128),
         rtol=3e-2, atol=3e-2),
    Case("tiny_bf16_8x8x8", 8, 8, 8, bf16, bf16, seed=11, block=(16, 16, 16)),
    Case("one_row_bf16_1x64x256", 1, 64, 256, bf16, bf16, seed=12, block=(16, 64, 64)),
]


def tolerance_ok(got: torch.Tensor, want: torch.Tensor, rtol: float, atol: float) -> tuple[bool, float]:
    got64, want64 = got.double(), want.double()
    diff = (got64 - want64).abs()
    ok = bool((diff <= atol + rtol * want64.abs()).all())
    return ok, float(diff.max()) if diff.numel() else 0.0
