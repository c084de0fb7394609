"""Launch-bound loops are meant to be captured in CUDA graphs: the launch entry points make no allocation and no
synchronisation once a plan (or, for attention, the first call of a shape) exists. A decode-shaped tt.dot and an
attention forward are captured, replayed, and must reproduce the eager results bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu

bf16, f16 = torch.bfloat16, torch.float16


def test_decode_dot_in_a_cuda_graph(built_libs, cuda_device):
    from triton_ext_b200 import backend as B
    dev = cuda_device
    g = torch.Generator().manual_seed(3)
    x = torch.randn(16, 4096, generator=g).to(bf16).to(dev)
    ws = [(torch.randn(4096, 1024, generator=g) * 0.02).to(bf16).to(dev) for _ in range(6)]
    plan = B.DotPlan(B.make_problem(16, 1024, 4096, bf16, bf16), None)
    eager = [torch.empty(16, 1024, dtype=bf16, device=dev) for _ in ws]
    for w, o in zip(ws, eager):
        plan.run(x, w, o)
    plan.check()
    outs = [torch.zeros_like(o) for o in eager]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for w, o in zip(ws, outs):
            plan.run(x, w, o)           # current stream = the capturing stream
    for replay in range(2):
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for o, e in zip(outs, eager):
            assert torch.equal(o, e), f"replay {replay}"
    plan.check()
    plan.close()


def test_attention_in_a_cuda_graph(built_libs, cuda_device):
    from triton_ext_b200 import attention as A
    dev = cuda_device
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.empty((2, 4, 512, 64)).normal_(0.0, 0.5, generator=g).to(f16).to(dev) for _ in range(3))
    eager = A.attention_forward(q, k, v, True, 0.5, check=True)   # also sizes the library's per-device scratch
    out = torch.zeros_like(eager)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(3):
            A.attention_forward(q, k, v, True, 0.5, out=out)
    graph.replay()
    torch.cuda.synchronize()
    A.check()
    assert torch.equal(out, eager)
