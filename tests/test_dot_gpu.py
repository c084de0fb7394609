"""Parity of the CUDA kernels with the oracle, through the C-ABI (ctypes -> libb200_dot.so).

Tolerances are north_star's: rtol = atol = 1e-2 for f16/bf16, 3e-2 for scaled fp8. The interpreter
oracle truncates fp32->bf16 where the kernels round to nearest even, so bf16 outputs are never compared
bit for bit with the oracle; bit-exact checks are made only between runs of the kernels themselves.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from tests.cases import (CFG1, CFG2, CFG3, CFG4, CFG5, GOLDEN_CASES, Case, make_inputs, reference_fp64, tolerance_ok)
from tests.test_oracle import DTYPE_CODE, c_oracle, golden_tensor

pytestmark = pytest.mark.gpu

bf16, f16, f8, f32 = torch.bfloat16, torch.float16, torch.float8_e4m3fn, torch.float32


@pytest.fixture(scope="module")
def B(built_libs, cuda_device):
    from triton_ext_b200 import backend
    assert backend.load_library().tx_dot_device_count() >= 1
    return backend


@pytest.fixture(scope="module")
def dot_lib(built_libs):
    lib = ctypes.CDLL(built_libs["oracles"]["libdot_oracle.so"])
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    lib.dot_oracle_tiles.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i64, i64,
                                     ctypes.c_float, i32, i32, i32, i32, vp, i32]
    lib.dot_oracle_tiles.restype = ctypes.c_int
    return lib


def gpu_dot(B, case, a, b, rs, cs, config=None):
    dev = torch.device("cuda:0")
    ad, bd = a.to(dev), b.to(dev)          # .to() keeps strides, so transposed layouts survive
    out = B.dot(ad, bd, out_dtype=case.out_dtype, row_scale=rs.to(dev) if rs is not None else None,
                col_scale=cs.to(dev) if cs is not None else None, alpha=case.alpha, config=config, check=True)
    return out.cpu()


def bits(t):
    return t.contiguous().view(torch.int32 if t.dtype == torch.float32 else torch.int16)


# ---- 1. every golden case: kernels vs committed oracle output vs exact arithmetic ---------------------------
@pytest.mark.parametrize("case", GOLDEN_CASES, ids=lambda c: c.name)
def test_golden_cases(B, case):
    launches = B.kernel_launches()
    a, b, rs, cs = make_inputs(case)
    got = gpu_dot(B, case, a, b, rs, cs)
    assert B.kernel_launches() > launches, "no kernel of this library was launched"
    want = golden_tensor(case.name, case.out_dtype)
    ok, err = tolerance_ok(got, want, case.rtol, case.atol)
    assert ok, f"vs oracle fixture: max err {err}"
    ok, err = tolerance_ok(got, reference_fp64(case, a, b, rs, cs), case.rtol, case.atol)
    assert ok, f"vs fp64: max err {err}"


# ---- 2. shape sweep against the C oracle (edges: 1, sub-tile, tile +- 1, ragged K) ---------------------------
SWEEP = [(1, 8, 8), (7, 16, 24), (8, 8, 8), (63, 64, 72), (64, 64, 64), (65, 72, 136), (127, 128, 120),
         (128, 128, 128), (129, 136, 200), (255, 264, 72), (256, 512, 320), (300, 520, 1000), (513, 40, 264)]


@pytest.mark.parametrize("m,n,k", SWEEP)
@pytest.mark.parametrize("dt", [bf16, f16, f8])
def test_shape_sweep(B, dot_lib, m, n, k, dt):
    if dt == f8 and (k % 16 or n % 16):
        # fp8 rows of A (K bytes) or of B (N bytes) that are not 16-byte multiples cannot be described to TMA:
        # the documented answer is TXD_ERR_UNSUPPORTED at plan creation, not a wrong result
        dev = torch.device("cuda:0")
        with pytest.raises(B.DotError) as e:
            B.dot(torch.zeros(m, k, device=dev).to(f8), torch.zeros(k, n, device=dev).to(f8), out_dtype=bf16)
        assert e.value.status == B.TXD_ERR_UNSUPPORTED
        return
    case = Case(f"sweep_{m}x{n}x{k}", m, n, k, dt, bf16 if dt == f8 else dt, seed=100 + m + n + k,
                scales=(dt == f8), block=(64, 64, 64), rtol=3e-2 if dt == f8 else 1e-2, atol=3e-2 if dt == f8 else 1e-2)
    a, b, rs, cs = make_inputs(case)
    got = gpu_dot(B, case, a, b, rs, cs)
    want = c_oracle(dot_lib, case, a, b, rs, cs, bf16_truncate=False)
    ok, err = tolerance_ok(got, want, case.rtol, case.atol)
    assert ok, f"max err {err}"


# ---- 3. every kernel configuration on one problem ------------------------------------------------------------
CONFIGS = [
    dict(block_n=256, cta_pair=1), dict(block_n=128, cta_pair=1), dict(block_n=256, cta_pair=1, stages=3, group_m=1),
    dict(block_n=256, cta_pair=2, schedule=1), dict(block_n=128, cta_pair=2, schedule=1), dict(block_n=64, cta_pair=2, schedule=1),
    dict(block_n=32, cta_pair=2, schedule=1), dict(block_n=16, cta_pair=2, schedule=1),
    dict(block_n=256, cta_pair=2, schedule=2), dict(block_n=64, cta_pair=2, schedule=2, max_ctas=37),
    dict(swap_ab=1, block_n=128, cta_pair=2, schedule=1), dict(swap_ab=1, block_n=16, cta_pair=2, schedule=2),
    dict(block_n=128, cta_pair=2, schedule=1, stages=2), dict(block_n=256, cta_pair=1, max_ctas=6),
    dict(block_n=256, cta_pair=1, schedule=3, max_ctas=10), dict(block_n=128, cta_pair=1, schedule=2), dict(block_n=64, cta_pair=2, schedule=3, max_ctas=50),
    dict(block_n=256, cta_pair=1, atoms=2), dict(block_n=64, cta_pair=2, schedule=2, atoms=2),
    # the wide pair tile (256 x 512: two 256-column MMA halves per K block)
    dict(block_n=512, cta_pair=1), dict(block_n=512, cta_pair=1, stages=2, group_m=1), dict(block_n=512, cta_pair=1, max_ctas=4),
]


@pytest.mark.parametrize("kw", CONFIGS, ids=lambda kw: ",".join(f"{k}={v}" for k, v in kw.items()))
@pytest.mark.parametrize("layout", ["row,row", "row,col", "col,row", "col,col"])
def test_config_sweep(B, dot_lib, kw, layout):
    la, lb = layout.split(",")
    case = Case("cfgsweep", 520, 776, 1096, bf16, bf16, seed=21, a_t=(la == "col"), b_t=(lb == "col"), block=(64, 64, 64))
    a, b, rs, cs = make_inputs(case)
    got = gpu_dot(B, case, a, b, rs, cs, config=B.make_config(**kw))
    want = c_oracle(dot_lib, case, a, b, rs, cs, bf16_truncate=False)
    ok, err = tolerance_ok(got, want, case.rtol, case.atol)
    assert ok, f"max err {err}"


# ---- 4. BASELINE configurations at full size --------------------------------------------------------------------
def check_full_size(B, dot_lib, case, n_c_tiles, n_interp_tiles, config=None):
    from oracle.interp_dot import interp_dot, sample_tiles, tile_mask
    a, b, rs, cs = make_inputs(case)
    got = gpu_dot(B, case, a, b, rs, cs, config=config)
    bm, bn, bk = case.block
    ids = sample_tiles(case.m, case.n, bm, bn, n_c_tiles, seed=case.seed)
    want = c_oracle(dot_lib, case, a, b, rs, cs, bf16_truncate=False, tile_ids=ids)
    mask = tile_mask(case.m, case.n, bm, bn, ids)
    ok, err = tolerance_ok(got[mask], want[mask], case.rtol, case.atol)
    assert ok, f"vs C oracle on {len(ids)} tiles: max err {err}"
    ids2 = ids[:n_interp_tiles]
    y = interp_dot(a, b, out_dtype=case.out_dtype, block_m=bm, block_n=bn, block_k=bk, row_scale=rs, col_scale=cs,
                   alpha=case.alpha, tile_ids=ids2)
    mask2 = tile_mask(case.m, case.n, bm, bn, ids2)
    ok, err = tolerance_ok(got[mask2], y[mask2], case.rtol, case.atol)
    assert ok, f"vs interpreter oracle on {len(ids2)} tiles: max err {err}"
    return a, b, rs, cs, got


def test_cfg1_fp16_512(B, dot_lib):
    a, b, rs, cs, got = check_full_size(B, dot_lib, CFG1, 64, 8)
    want = golden_tensor(CFG1.name, f16)          # fp16 casts round the same way on both sides:
    assert float((bits(got) != bits(want)).float().mean()) < 0.02  # only fp32 summation order differs


def test_cfg2_loop_split_tail(B, dot_lib):
    cfg = B.make_config(k_split_point=4096)       # BLOCK_K = 128: main [0, 4096), 64-wide remainder
    a, b, rs, cs, got = check_full_size(B, dot_lib, CFG2, 12, 2, config=cfg)
    check_whole_matrix(CFG2, a, b, rs, cs, got)
    dev = torch.device("cuda:0")
    ad, bd = a.to(dev), b.to(dev)
    # the split point never changes a bit of the result
    for split in (0, -1, 2048, 4160 // 64 * 64):
        other = B.dot(ad, bd, out_dtype=bf16, config=B.make_config(k_split_point=split), check=True).cpu()
        assert torch.equal(bits(other), bits(got)), f"k_split_point={split}"
    # linearity in a power-of-two alpha is exact
    twice = B.dot(ad, bd, out_dtype=bf16, alpha=2.0, check=True).cpu()
    assert torch.equal(bits(twice), bits((got.float() * 2).to(bf16)))
    # (A B)^T = B^T A^T: swapping the operand roles accumulates in the same k order
    swapped = B.dot(bd.t(), ad.t(), out_dtype=bf16, check=True).cpu()
    assert torch.equal(bits(swapped.t().contiguous()), bits(got))
    # pair / single / stream-K / one K atom per stage / the wide tile agree within tolerance (partial sums are formed
    # in a different order)
    for kw in (dict(cta_pair=2, schedule=1), dict(cta_pair=2, schedule=2), dict(atoms=1), dict(block_n=512, cta_pair=1)):
        other = B.dot(ad, bd, out_dtype=bf16, config=B.make_config(**kw), check=True).cpu()
        ok, err = tolerance_ok(other, got, 1e-2, 1e-2)
        assert ok, (kw, err)


def test_cfg3_decode_skinny(B, dot_lib):
    a, b, rs, cs, got = check_full_size(B, dot_lib, CFG3, 112, 4)
    dev = torch.device("cuda:0")
    again = B.dot(a.to(dev), b.to(dev), out_dtype=bf16, check=True).cpu()
    assert torch.equal(bits(again), bits(got)), "two runs of one plan must agree bit for bit"


def check_whole_matrix(case, a, b, rs, cs, got):
    """The kernel's whole C against an fp32 matmul of the same, already quantised operands upcast to fp32, in row panels
    on the GPU (a checker: torch's fp32 GEMM with TF32 off). The oracle sample above pins the arithmetic on a few tiles;
    this pass covers every element, so a tile written to the wrong place anywhere in the raster cannot hide."""
    dev = torch.device("cuda:0")
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        b32 = b.to(dev).float()
        cs_d = cs.to(dev) if cs is not None else None
        worst = 0.0
        for r0 in range(0, case.m, 2048):
            r1 = min(r0 + 2048, case.m)
            ref = a[r0:r1].to(dev).float() @ b32 * case.alpha
            if rs is not None:
                ref = ref * rs[r0:r1].to(dev)[:, None] * cs_d[None, :]
            diff = (got[r0:r1].to(dev).float() - ref).abs()
            bad = diff > case.atol + case.rtol * ref.abs()
            assert not bool(bad.any()), f"rows {r0}..{r1}: {int(bad.sum())} elements off, max diff {float(diff.max())}"
            worst = max(worst, float(diff.max()))
        return worst
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_cfg4_fp8_scaled(B, dot_lib):
    a, b, rs, cs, got = check_full_size(B, dot_lib, CFG4, 6, 1)
    check_whole_matrix(CFG4, a, b, rs, cs, got)


def test_cfg5_big_bf16_and_n_shards(B, dot_lib):
    from triton_ext_b200.parallel import split_range
    a, b, rs, cs, got = check_full_size(B, dot_lib, CFG5, 4, 1)
    check_whole_matrix(CFG5, a, b, rs, cs, got)
    dev = torch.device("cuda:0")
    ad, bd = a.to(dev), b.to(dev)
    # an N-shard computed alone is bit-identical to the same columns of the unsharded result
    for world, rank in ((2, 1), (8, 5)):
        n0, n1 = split_range(CFG5.n, world, rank, align=256)
        panel = B.dot(ad, bd[:, n0:n1], out_dtype=bf16, check=True).cpu()
        assert torch.equal(bits(panel), bits(got[:, n0:n1].contiguous()))


# ---- 5. the host-buffer entry point ------------------------------------------------------------------------------
def test_run_host_matches_device_path(B):
    case = Case("host", 384, 520, 264, bf16, bf16, seed=31, scales=True)
    a, b, rs, cs = make_inputs(case)
    want = gpu_dot(B, case, a, b, rs, cs)
    plan = B.DotPlan(B.make_problem(case.m, case.n, case.k, bf16, bf16, row_scale=True, col_scale=True))
    out = torch.empty(case.m, case.n, dtype=bf16).pin_memory()
    for _ in range(2):
        out.zero_()
        plan.run_host(a.contiguous().pin_memory(), b.contiguous().pin_memory(), out, rs, cs)
        assert torch.equal(bits(out), bits(want))
    plan.close()


@pytest.mark.parametrize("m,n,a_col_major,b_col_major", [(2048, 4096, False, False), (3000, 4096, False, True),
                                                         (4096, 2048, False, False), (4096, 3000, False, True),
                                                         (2048, 4096, True, False), (2048, 3000, True, False),
                                                         (2048, 4096, True, True)])
def test_run_host_pipelined_panels(B, m, n, a_col_major, b_col_major):
    """Above 32 MB the host-buffer entry point cuts one operand and C into panels (rows of A and C when A is
    row-major and not the smaller operand, else columns of B and C: the smaller operand travels whole, first) and
    overlaps copy-in, kernel and copy-out on three streams. Same schedule forced on both paths: the panels must reproduce the one-launch
    result bit for bit (every output element sums the same K blocks in the same order)."""
    k = 4096            # every case moves more than 32 MB
    g = torch.Generator().manual_seed(77)
    a = torch.randn(m, k, generator=g).to(bf16)
    b = (torch.randn(k, n, generator=g) * 0.05).to(bf16)
    rs = torch.rand(m, generator=g) + 0.5
    cs = torch.rand(n, generator=g) + 0.5
    a_store = a.t().contiguous() if a_col_major else a          # [k, m] storage when column-major
    b_store = b.t().contiguous() if b_col_major else b          # [n, k] storage when column-major
    cfg = B.make_config(schedule=B.TXD_SCHED_DATA_PARALLEL)
    pr = B.make_problem(m, n, k, bf16, bf16, row_scale=True, col_scale=True,
                        a_layout=B.TXD_COL_MAJOR if a_col_major else B.TXD_ROW_MAJOR,
                        b_layout=B.TXD_COL_MAJOR if b_col_major else B.TXD_ROW_MAJOR)
    plan = B.DotPlan(pr, cfg)
    dev = torch.device("cuda:0")
    want = torch.empty(m, n, dtype=bf16, device=dev)
    plan.run(a_store.to(dev), b_store.to(dev), want, rs.to(dev), cs.to(dev))
    plan.check()
    out = torch.empty(m, n, dtype=bf16).pin_memory()
    for _ in range(2):
        out.zero_()
        plan.run_host(a_store.pin_memory(), b_store.pin_memory(), out, rs, cs)
        assert torch.equal(bits(out), bits(want.cpu()))
    ref = (a.float() @ b.float()) * rs[:, None] * cs[None, :]
    assert bool(((out.float() - ref).abs() <= 1e-2 + 1e-2 * ref.abs()).all())
    plan.close()


def test_empty_and_zero_k(B):
    dev = torch.device("cuda:0")
    out = B.dot(torch.zeros(0, 64, dtype=bf16, device=dev), torch.zeros(64, 32, dtype=bf16, device=dev), check=True)
    assert out.shape == (0, 32)
    out = torch.full((16, 24), 7.0, dtype=bf16, device=dev)
    B.dot(torch.zeros(16, 0, dtype=bf16, device=dev), torch.zeros(0, 24, dtype=bf16, device=dev), out=out, check=True)
    assert bool((out == 0).all())


def test_padded_leading_dimensions(B, dot_lib):
    dev = torch.device("cuda:0")
    case = Case("ld", 200, 136, 72, bf16, bf16, seed=41, block=(64, 64, 64))
    a, b, rs, cs = make_inputs(case)
    abig = torch.zeros(200, 96, dtype=bf16, device=dev)
    bbig = torch.zeros(72, 160, dtype=bf16, device=dev)
    cbig = torch.full((200, 144), 3.0, dtype=bf16, device=dev)
    abig[:, :72] = a.to(dev)
    bbig[:, :136] = b.to(dev)
    B.dot(abig[:, :72], bbig[:, :136], out=cbig[:, :136], check=True)
    want = c_oracle(dot_lib, case, a, b, None, None, bf16_truncate=False)
    ok, err = tolerance_ok(cbig[:, :136].cpu(), want, 1e-2, 1e-2)
    assert ok, err
    assert bool((cbig[:, 136:] == 3.0).all()), "columns outside C were written"


# ---- 6. the pass pipeline drives the kernels ---------------------------------------------------------------------
def test_pipeline_to_plan(B, dot_lib):
    from triton_ext_b200 import plugin as P
    case = Case("pipe", 512, 512, 1096, bf16, bf16, seed=51, block=(64, 64, 128))
    a, b, rs, cs = make_inputs(case)
    pr = B.make_problem(case.m, case.n, case.k, bf16, bf16)
    cfg, info, module = P.lower_dot(pr, 128)
    assert cfg.k_split_point == 1024 and info["k_main_iters"] * info["block_k"] == 1024 and info["k_tail_iters"] >= 1
    lib = B.load_library()
    lib.txir_module_create_plan.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)]
    h = ctypes.c_void_p()
    assert lib.txir_module_create_plan(module._h, 0, ctypes.byref(h)) == B.TXD_OK
    dev = torch.device("cuda:0")
    ad, bd = a.to(dev), b.to(dev)
    out = torch.empty(case.m, case.n, dtype=bf16, device=dev)
    s = torch.cuda.current_stream()
    assert lib.tx_dot_run(h, ad.data_ptr(), bd.data_ptr(), out.data_ptr(), None, None, ctypes.c_void_p(s.cuda_stream)) == B.TXD_OK
    assert lib.tx_dot_plan_check(h, ctypes.c_void_p(s.cuda_stream)) == B.TXD_OK
    lib.tx_dot_plan_destroy(h)
    want = c_oracle(dot_lib, case, a, b, None, None, bf16_truncate=False)
    ok, err = tolerance_ok(out.cpu(), want, 1e-2, 1e-2)
    assert ok, err


# ---- 7. a wait that runs out is reported, and the context stays usable ----------------------------------------
def test_bounded_wait_reports_timeout(B, monkeypatch):
    dev = torch.device("cuda:0")
    a = torch.randn(256, 512, device=dev).to(bf16)
    b = torch.randn(512, 256, device=dev).to(bf16)
    out = torch.empty(256, 256, dtype=bf16, device=dev)
    monkeypatch.setenv("TXD_INJECT_STALL", "1")    # the producer stops after its first K block
    monkeypatch.setenv("TXD_WAIT_LIMIT_MS", "50")
    plan = B.DotPlan(B.make_problem(256, 256, 512, bf16, bf16), B.make_config(cta_pair=2, schedule=1))
    monkeypatch.delenv("TXD_INJECT_STALL")
    monkeypatch.delenv("TXD_WAIT_LIMIT_MS")
    plan.run(a, b, out)
    with pytest.raises(B.DotError) as e:
        plan.check()
    assert e.value.status == B.TXD_ERR_DEVICE_TIMEOUT
    plan.close()
    # same context, healthy plan: still works
    good = B.dot(a, b, out_dtype=bf16, check=True)
    ref = a.float() @ b.float()
    assert bool(((good.float() - ref).abs() <= 1e-2 + 1e-2 * ref.abs()).all())


# ---- 8. K-sharded GEMM with the exchange in its epilogue, emulated on one GPU ----------------------------------
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("partial_dtype", [f32, bf16])
def test_slot_stores_and_reduction_single_gpu(B, dot_lib, partial_dtype, world):
    """`world` "ranks" share one GPU: each runs its K shard and stores tiles into its slot of the owner's buffer
    (all buffers are local here, on a real job they are peer-mapped); the slot reduction then gives each
    owner its rows of C. The kernels run one after the other, never waiting on one another."""
    dev = torch.device("cuda:0")
    case = Case("kshard", 256 * world, 384, 1152, bf16, bf16, seed=61, scales=True, block=(64, 64, 64))
    a, b, rs, cs = make_inputs(case)
    ad, bd, rsd, csd = a.to(dev), b.to(dev), rs.to(dev), cs.to(dev)
    rows = case.m // world
    slots = [torch.zeros(world, rows, case.n, dtype=partial_dtype, device=dev) for _ in range(world)]
    ptrs = [t.data_ptr() for t in slots]
    kshard = case.k // world
    for rank in range(world):
        plan = B.DotPlan(B.make_problem(case.m, case.n, kshard, bf16, partial_dtype, lda=case.k),  # A shard is a column slice
                         B.make_config(schedule=B.TXD_SCHED_DATA_PARALLEL, swap_ab=2, cta_pair=1, block_n=128))
        a_sh = ad[:, rank * kshard:(rank + 1) * kshard]
        b_sh = bd[rank * kshard:(rank + 1) * kshard, :]
        plan.run_to_slots(a_sh, b_sh, ptrs, rank)
        plan.check()
        plan.close()
    want = c_oracle(dot_lib, case, a, b, rs, cs, bf16_truncate=False)
    for owner in range(world):
        out = torch.empty(rows, case.n, dtype=bf16, device=dev)
        B.reduce_slots(slots[owner], out, row_scale=rsd[owner * rows:(owner + 1) * rows], col_scale=csd)
        torch.cuda.synchronize()
        got = out.cpu().double()
        w = want[owner * rows:(owner + 1) * rows].double()
        bound = 1e-2 + 1e-2 * w.abs()
        if partial_dtype == bf16:
            # each partial is rounded to bf16 before the sum: allow one bf16 ulp of every partial's magnitude
            sl = slice(owner * rows, (owner + 1) * rows)
            mag = sum((a[sl, r * kshard:(r + 1) * kshard].double() @ b[r * kshard:(r + 1) * kshard].double()).abs()
                      for r in range(world))
            bound = bound + 2.0 ** -8 * mag * rs[sl].double()[:, None] * cs.double()[None, :]
        assert bool(((got - w).abs() <= bound).all()), (owner, float((got - w).abs().max()))
    # argument checks of the slot form
    plan = B.DotPlan(B.make_problem(case.m, case.n, kshard, bf16, f32, row_scale=True))
    with pytest.raises(B.DotError):
        plan.run_to_slots(ad[:, :kshard], bd[:kshard], ptrs, 0)
    plan.close()


@pytest.mark.parametrize("world,rows,n", [(3, 37, 1001), (2, 5, 7), (4, 64, 1004), (8, 33, 520), (8, 256, 4096)])
@pytest.mark.parametrize("slot_dtype", [f32, bf16])
def test_slot_reduction_shapes(B, world, rows, n, slot_dtype):
    """The slot sum on its own: any slot count, ragged and vector-width row lengths, every output type, a padded
    output; summed in slot order in fp32 (bit-exact against the same sum written with torch for fp32 output)."""
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(world * 1000 + n)
    slots = torch.randn(world, rows, n, generator=g).to(slot_dtype).to(dev)
    rs = (torch.rand(rows, generator=g) + 0.5).to(dev)
    cs = (torch.rand(n, generator=g) + 0.5).to(dev)
    acc = torch.zeros(rows, n, device=dev)
    for s in range(world):
        acc = acc + slots[s].float()
    for out_dtype in (f32, bf16, f16):
        padded = torch.full((rows, n + 3), 7.0, device=dev, dtype=out_dtype)
        out = padded[:, :n]
        B.reduce_slots(slots, out, row_scale=rs, col_scale=cs, alpha=0.5)
        torch.cuda.synchronize()
        want = (acc * (rs * 0.5)[:, None] * cs[None, :])
        if out_dtype == f32:
            assert torch.equal(out, want)
        else:
            assert torch.equal(out, want.to(out_dtype))
        assert bool((padded[:, n:] == 7.0).all())


def test_slot_exchange_in_pieces_single_gpu(B):
    """The exchange cut into pieces: piece j of every rank fills rows [j, j + 1) * rows / parts of its slot in every
    owner's buffer and nothing else, all pieces together give the slots of the one-piece form bit for bit, and the
    piecewise sums give the one-piece result bit for bit."""
    dev = torch.device("cuda:0")
    world, parts = 2, 2
    case = Case("kshard_pieces", 1024, 384, 1152, bf16, bf16, seed=62, scales=True, block=(64, 64, 64))
    a, b, rs, cs = make_inputs(case)
    ad, bd, rsd, csd = a.to(dev), b.to(dev), rs.to(dev), cs.to(dev)
    rows, kshard = case.m // world, case.k // world
    cfg = dict(schedule=B.TXD_SCHED_DATA_PARALLEL, swap_ab=2, cta_pair=1, block_n=128)
    plans = [B.DotPlan(B.make_problem(case.m, case.n, kshard, bf16, f32, lda=case.k), B.make_config(**cfg)) for _ in range(world)]
    shards = [(ad[:, r * kshard:(r + 1) * kshard], bd[r * kshard:(r + 1) * kshard, :]) for r in range(world)]
    whole = [torch.zeros(world, rows, case.n, dtype=f32, device=dev) for _ in range(world)]
    for r in range(world):
        plans[r].run_to_slots(*shards[r], [t.data_ptr() for t in whole], r)
    pieces = [torch.full((world, rows, case.n), float("nan"), dtype=f32, device=dev) for _ in range(world)]
    ptrs = [t.data_ptr() for t in pieces]
    outs = [torch.zeros(rows, case.n, dtype=bf16, device=dev) for _ in range(world)]
    per = rows // parts
    for j in range(parts):
        for r in range(world):
            plans[r].run_to_slots(*shards[r], ptrs, r, part=j, parts=parts)
        torch.cuda.synchronize()
        for owner in range(world):
            written = ~torch.isnan(pieces[owner])
            assert bool(written[:, :(j + 1) * per].all()) and not bool(written[:, (j + 1) * per:].any()), (j, owner)
            B.reduce_slots(pieces[owner], outs[owner], row_scale=rsd[owner * rows:(owner + 1) * rows], col_scale=csd,
                           row0=j * per, rows=per)
    torch.cuda.synchronize()
    for r in range(world):
        plans[r].check()
    for owner in range(world):
        assert torch.equal(pieces[owner], whole[owner])
        ref = torch.empty(rows, case.n, dtype=bf16, device=dev)
        B.reduce_slots(whole[owner], ref, row_scale=rsd[owner * rows:(owner + 1) * rows], col_scale=csd)
        assert torch.equal(outs[owner], ref)
    with pytest.raises(B.DotError):
        plans[0].run_to_slots(*shards[0], ptrs, 0, part=0, parts=3)   # 2 tile rows per rank do not divide into 3
    with pytest.raises(B.DotError):
        B.reduce_slots(pieces[0], outs[0], row0=rows - 8, rows=16)
    for pl in plans:
        pl.close()
