"""tx_dot_run_static_scratch: the launch for callers that cannot allocate device memory (a host whose
memory pool is owned by another library, a thread that must not take the allocator lock, a sandbox that
forbids cudaMalloc). Its stream-K scratch is a fixed array inside the library instead of a cudaMalloc'ed
buffer, so the test checks three things through the C-ABI:

  * its output equals the plan-based entry point's (same kernel, same schedule) on two calls in a row —
    the second call finds the array as the first one left it;
  * no device memory is taken by the calls (free memory before == after, once the first call has done
    the per-device set-up);
  * a configuration whose scratch does not fit the array is refused with a clear error.

Collected last on purpose: if it fails, a run that stops at the first failure has already run the rest.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

bf16 = torch.bfloat16


@pytest.fixture(scope="module")
def B(built_libs, cuda_device):
    from triton_ext_b200 import backend
    lib = backend.load_library()
    vp = ctypes.c_void_p
    lib.tx_dot_run_static_scratch.argtypes = [ctypes.POINTER(backend.Problem), ctypes.POINTER(backend.Config),
                                              vp, vp, vp, vp, vp, vp]
    lib.tx_dot_run_static_scratch.restype = ctypes.c_int
    lib.tx_dot_static_scratch_check.argtypes = [vp]
    lib.tx_dot_static_scratch_check.restype = ctypes.c_int
    lib.tx_dot_static_scratch_capacity.restype = ctypes.c_int64
    lib.tx_dot_static_scratch_last_error.restype = ctypes.c_char_p
    return backend


def run_static(B, pr, cfg, a, b, c, rs=None, cs=None):
    lib = B.load_library()
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.tx_dot_run_static_scratch(ctypes.byref(pr), ctypes.byref(cfg) if cfg is not None else None,
                                       a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                       rs.data_ptr() if rs is not None else None,
                                       cs.data_ptr() if cs is not None else None, s)
    assert rc == B.TXD_OK, lib.tx_dot_static_scratch_last_error().decode()
    assert lib.tx_dot_static_scratch_check(s) == B.TXD_OK, lib.tx_dot_static_scratch_last_error().decode()


CASES = [
    # m, n, k, config for both entry points                      (what it exercises)
    (16, 4096, 1024, dict(swap_ab=1, block_n=16)),               # decode shape, swapped roles, many partial tiles
    (520, 776, 1096, dict(block_n=32, max_ctas=100)),            # ragged edges, K remainder, direct + fix-up stores
    (512, 512, 4160, dict(block_n=64, max_ctas=60)),             # TMA-store epilogue for whole tiles
]


@pytest.mark.parametrize("m,n,k,kw", CASES)
def test_matches_plan_entry_point_twice_without_allocating(B, m, n, k, kw):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(7)
    a = torch.randn(m, k, generator=g).to(bf16).to(dev)
    b = (torch.randn(k, n, generator=g) * 0.1).to(bf16).to(dev)
    rs = (torch.rand(m, generator=g) + 0.5).to(dev)
    cs = (torch.rand(n, generator=g) + 0.5).to(dev)
    pr = B.make_problem(m, n, k, bf16, bf16, row_scale=True, col_scale=True)
    cfg = B.make_config(schedule=B.TXD_SCHED_STREAM_K, cta_pair=2, **kw)
    want = torch.empty(m, n, dtype=bf16, device=dev)
    plan = B.DotPlan(pr, cfg)
    assert plan.info["schedule"] == B.TXD_SCHED_STREAM_K and plan.info["scratch_bytes"] > 0
    plan.run(a, b, want, rs, cs)
    plan.check()
    plan.close()
    ref = (a.float() @ b.float()) * rs[:, None] * cs[None, :]
    assert bool(((want.float() - ref).abs() <= 1e-2 + 1e-2 * ref.abs()).all())

    got = torch.empty(m, n, dtype=bf16, device=dev)
    run_static(B, pr, cfg, a, b, got, rs, cs)        # first call: also does the per-device set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    for call in range(2):
        got.fill_(float("nan"))
        run_static(B, pr, cfg, a, b, got, rs, cs)
        diff = (got.float() - want.float()).abs()
        assert bool((diff <= 1e-2 + 1e-2 * want.float().abs()).all()), f"call {call}: max diff {float(diff.max())}"
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}: same kernel, same bits expected"
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before, "the static-scratch entry point took device memory"


def test_oversized_scratch_is_refused(B):
    dev = torch.device("cuda:0")
    lib = B.load_library()
    cap = lib.tx_dot_static_scratch_capacity()
    assert cap == 4 << 20
    m = n = k = 2048
    a = torch.zeros(m, k, dtype=bf16, device=dev)
    out = torch.empty(m, n, dtype=bf16, device=dev)
    pr = B.make_problem(m, n, k, bf16, bf16)
    cfg = B.make_config(block_n=256)  # 148 CTAs * 2 * 256 * 128 * 4 B = 38.8 MB of partial tiles
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.tx_dot_run_static_scratch(ctypes.byref(pr), ctypes.byref(cfg), a.data_ptr(), a.data_ptr(), out.data_ptr(),
                                       None, None, s)
    assert rc == B.TXD_ERR_UNSUPPORTED
    msg = lib.tx_dot_static_scratch_last_error().decode()
    assert "exceeds the static scratch" in msg and str(cap) in msg
    # the same problem fits once the grid is capped: 15 CTAs * 2 * 256 * 128 * 4 B = 3.9 MB
    cfg = B.make_config(block_n=256, max_ctas=15)
    b = torch.zeros(k, n, dtype=bf16, device=dev)
    run_static(B, pr, cfg, a, b, out)
    assert bool((out == 0).all())


def test_static_entry_reports_a_wait_that_runs_out_and_recovers(B, monkeypatch):
    """The status word of the static entry point lives inside the fixed array: a wait that runs out (the producer is
    stalled from the host, no GPU fault is involved) must be reported by tx_dot_static_scratch_check, cleared, and a
    healthy call on the same array straight afterwards must give the exact result."""
    dev = torch.device("cuda:0")
    lib = B.load_library()
    m, n, k = 256, 512, 1024
    g = torch.Generator().manual_seed(9)
    a = torch.randn(m, k, generator=g).to(bf16).to(dev)
    b = torch.randn(k, n, generator=g).to(bf16).to(dev)
    out = torch.empty(m, n, dtype=bf16, device=dev)
    pr = B.make_problem(m, n, k, bf16, bf16)
    cfg = B.make_config(block_n=64, max_ctas=24)
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    monkeypatch.setenv("TXD_INJECT_STALL", "1")    # read by every launch of this entry point
    monkeypatch.setenv("TXD_WAIT_LIMIT_MS", "50")
    rc = lib.tx_dot_run_static_scratch(ctypes.byref(pr), ctypes.byref(cfg), a.data_ptr(), b.data_ptr(), out.data_ptr(), None, None, s)
    assert rc == B.TXD_OK
    assert lib.tx_dot_static_scratch_check(s) == B.TXD_ERR_DEVICE_TIMEOUT
    assert "wait ran out" in lib.tx_dot_static_scratch_last_error().decode()
    monkeypatch.delenv("TXD_INJECT_STALL")
    monkeypatch.delenv("TXD_WAIT_LIMIT_MS")
    assert lib.tx_dot_static_scratch_check(s) == B.TXD_OK          # the status word was cleared by the report
    want = B.dot(a, b, out_dtype=bf16, config=B.make_config(schedule=B.TXD_SCHED_STREAM_K, cta_pair=2, block_n=64, max_ctas=24), check=True)
    out.fill_(float("nan"))
    run_static(B, pr, cfg, a, b, out)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
