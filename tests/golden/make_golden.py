"""Generate tests/golden/dot_golden.npz: the interpreter oracle's output for every case of
tests/cases.py:GOLDEN_CASES, stored as raw bit patterns (uint16 for f16/bf16, uint32 for f32).

Run from the repository root:   python tests/golden/make_golden.py
Needs only torch + triton (CPU); inputs are regenerated from the seeds, so they are not stored.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.interp_dot import interp_dot  # noqa: E402
from tests.cases import GOLDEN_CASES, make_inputs  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.float32:
        return t.contiguous().view(torch.int32).numpy().astype(np.uint32)
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def main():
    out = {}
    for c in GOLDEN_CASES:
        a, b, rs, cs = make_inputs(c)
        bm, bn, bk = c.block
        y = interp_dot(a, b, out_dtype=c.out_dtype, block_m=bm, block_n=bn, block_k=bk, row_scale=rs, col_scale=cs,
                       alpha=c.alpha)
        out[c.name] = bits(y)
        print(f"{c.name}: {tuple(y.shape)} {y.dtype}", flush=True)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dot_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
