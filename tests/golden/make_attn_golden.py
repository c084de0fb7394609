"""Generates tests/golden/attn_golden.npz by running the reference's own forward kernel on the CPU.

The reference's `_attn_fwd` (pass/LoopSplit/06-fused-attention.py:164-240) is executed by Triton's
interpreter (TRITON_INTERPRET=1) on CPU tensors. The reference file cannot be imported as it stands on a
machine without a GPU (it asks the driver for the active device and its capability at import time,
:28-41,:268), so its source text is read from the reference checkout, those three queries are answered
with constants in memory, and the module is executed from that text. Nothing of it is written anywhere.

Run in a container that has the reference checked out:
    python tests/golden/make_attn_golden.py /path/to/reference
The inputs follow the reference's test (`test_op`, :690-695): seed 20, normal(0, 0.5), fp16, sm_scale 0.5; the fp8
cases cast them to float8_e5m2 the way the reference's benchmark does (:774-779).
"""
import linecache
import os
import re
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402

# name: (Z, H, N_CTX, HEAD_DIM, causal, BLOCK_M, BLOCK_N)
CASES = {
    "causal_d64": (1, 2, 256, 64, True, 64, 32),
    "full_d64": (1, 2, 256, 64, False, 64, 32),
    "causal_d128_n384": (1, 1, 384, 128, True, 128, 64),
    "full_d128": (2, 1, 128, 128, False, 64, 64),
    # the narrow heads of the reference's domain (HEAD_DIM in {16, 32, 64, 128, 256}, :589)
    "causal_d32": (1, 2, 256, 32, True, 64, 32),
    "full_d16": (1, 2, 256, 16, False, 64, 16),      # the kernel asserts BLOCK_N <= HEAD_DIM (:175)
    "causal_d256": (1, 1, 256, 256, True, 64, 64),
}
# the fp8 forward (q, k, v, out float8_e5m2, V laid out with N_CTX contiguous, P rounded to e5m2; :81-82, :191, :774-779)
FP8_CASES = {
    "fp8_causal_d64": (1, 2, 256, 64, True, 64, 32),
    "fp8_full_d128": (1, 1, 256, 128, False, 64, 64),
}
SM_SCALE = 0.5
# name: (Z, H, N_CTX, HEAD_DIM, causal); the reference's backward asserts N_CTX % 128 == 0 and is causal-only
BWD_CASES = {
    "bwd_causal_d64": (1, 2, 256, 64, True),
    "bwd_causal_d128": (1, 1, 256, 128, True),
    "bwd_causal_d256": (1, 1, 128, 256, True),
    "bwd_causal_d32": (1, 2, 256, 32, True),   # HEAD_DIM 16 has no forward configuration with BLOCK_N <= HEAD_DIM in the
                                               # reference's autotuning list, so its autograd function cannot run there
}


def load_reference(root: str):
    path = os.path.join(root, "pass", "LoopSplit", "06-fused-attention.py")
    src = open(path).read()
    src = src.replace("DEVICE = triton.runtime.driver.active.get_active_torch_device()", 'DEVICE = "cpu"')
    src = re.sub(r"def is_hip\(\):\n    return .*\n", "def is_hip():\n    return False\n", src)
    src = re.sub(r"def is_cuda\(\):\n    return .*\n", "def is_cuda():\n    return False\n", src)
    src = src.replace("torch.cuda.get_device_capability()", "(0, 0)")
    mod = types.ModuleType("reference_fused_attention")
    mod.__file__ = path
    linecache.cache[path] = (len(src), None, src.splitlines(True), path)  # the interpreter reads kernel source by file name
    exec(compile(src, path, "exec"), mod.__dict__)
    return mod


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRITON_EXT_REFERENCE", "")
    if not root or not os.path.isdir(root):
        raise SystemExit("usage: make_attn_golden.py <reference checkout>")
    mod = load_reference(root)
    kernel = mod._attn_fwd.fn  # below the autotuner: the block sizes are given explicitly
    out = {}
    for name, (z, h, n, d, causal, bm, bn) in CASES.items():
        torch.manual_seed(20)
        q = torch.empty((z, h, n, d), dtype=torch.float16).normal_(mean=0.0, std=0.5)
        k = torch.empty((z, h, n, d), dtype=torch.float16).normal_(mean=0.0, std=0.5)
        v = torch.empty((z, h, n, d), dtype=torch.float16).normal_(mean=0.0, std=0.5)
        o = torch.empty_like(q)
        m = torch.empty((z, h, n), dtype=torch.float32)
        grid = (triton.cdiv(n, bm), z * h, 1)
        kernel[grid](q, k, v, SM_SCALE, m, o, *q.stride(), *k.stride(), *v.stride(), *o.stride(), z, h, N_CTX=n,
                     HEAD_DIM=d, BLOCK_M=bm, BLOCK_N=bn, CAUSAL=causal)
        for key, t in (("q", q), ("k", k), ("v", v), ("o", o)):
            out[f"{name}.{key}"] = t.numpy().view(np.uint16)  # fp16 bit patterns
        out[f"{name}.m"] = m.numpy()
        out[f"{name}.meta"] = np.array([z, h, n, d, int(causal), bm, bn], dtype=np.int32)
        print(name, "done", flush=True)
    for name, (z, h, n, d, causal, bm, bn) in FP8_CASES.items():
        torch.manual_seed(20)
        q, k, v = (torch.empty((z, h, n, d), dtype=torch.float16).normal_(mean=0.0, std=0.5) for _ in range(3))
        q, k = q.to(torch.float8_e5m2), k.to(torch.float8_e5m2)
        v = v.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2).to(torch.float8_e5m2)  # as the reference's benchmark does
        o = torch.empty_like(q)
        m = torch.empty((z, h, n), dtype=torch.float32)
        grid = (triton.cdiv(n, bm), z * h, 1)
        kernel[grid](q, k, v, SM_SCALE, m, o, *q.stride(), *k.stride(), *v.stride(), *o.stride(), z, h, N_CTX=n,
                     HEAD_DIM=d, BLOCK_M=bm, BLOCK_N=bn, CAUSAL=causal)
        for key, t in (("q", q), ("k", k), ("v", v), ("o", o)):
            out[f"{name}.{key}"] = t.contiguous().view(torch.uint8).numpy()  # e5m2 bytes, logical [Z, H, N_CTX, HEAD_DIM] order
        out[f"{name}.m"] = m.numpy()
        out[f"{name}.meta"] = np.array([z, h, n, d, int(causal), bm, bn], dtype=np.int32)
        print(name, "done", flush=True)
    # forward + backward through the reference's autograd function (`attention = _attention.apply`, :690). With a
    # single autotuning configuration the autotuner does not try to time kernels on a device.
    all_configs = list(mod._attn_fwd.configs)
    for name, (z, h, n, d, causal) in BWD_CASES.items():
        mod._attn_fwd.configs = [c for c in all_configs if c.kwargs["BLOCK_N"] <= d][:1]
        mod._attn_fwd.cache.clear()
        torch.manual_seed(20)
        q, k, v = (torch.empty((z, h, n, d), dtype=torch.float16).normal_(mean=0.0, std=0.5).requires_grad_() for _ in range(3))
        d_o = torch.randn_like(q)
        o = mod.attention(q, k, v, causal, SM_SCALE)
        o.backward(d_o)
        for key, t in (("q", q), ("k", k), ("v", v), ("o", o), ("do", d_o), ("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
            out[f"{name}.{key}"] = t.detach().numpy().view(np.uint16)
        out[f"{name}.meta"] = np.array([z, h, n, d, int(causal)], dtype=np.int32)
        print(name, "done", flush=True)
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")
    np.savez_compressed(dst, sm_scale=np.float32(SM_SCALE), **out)
    print(dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
