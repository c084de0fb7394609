"""loop_split: the product pass against (a) the known answers of the reference's lit test
pass/LoopSplit/test/loop-split.mlir, (b) the C restatement of LoopSplit.cpp (oracle/loop_split_oracle.c)
in "as-written" mode, and (c) meaning preservation in "intent" mode."""
import ctypes
import itertools
import os
import random

import pytest

from triton_ext_b200 import plugin as P

ORACLE_PRED = {"slt": 0, "sle": 1, "sgt": 2, "sge": 3, "ult": 4, "ule": 5, "ugt": 6, "uge": 7}


class LsResult(ctypes.Structure):
    _fields_ = [("split", ctypes.c_int32), ("mid", ctypes.c_int32), ("cmp1", ctypes.c_int32), ("cmp2", ctypes.c_int32)]


@pytest.fixture(scope="module")
def oracle(built_libs):
    lib = ctypes.CDLL(built_libs["oracles"]["libloop_split_oracle.so"])
    lib.ls_bisect_as_written.argtypes = [ctypes.c_int32] * 8 + [ctypes.POINTER(LsResult)]
    lib.ls_run_original.argtypes = [ctypes.c_int32] * 6
    lib.ls_run_original.restype = ctypes.c_int64
    return lib


def run_pass(loop, mode):
    P.load_default_plugins()
    m = P.Module()
    m.set_attr("loop_split.mode", mode)
    idx = m.add_loop(loop)
    before = m.simulate(idx)
    pm = P.PassManager()
    assert pm.add("loop_split") == P.TP_SUCCESS
    assert pm.run(m) == 0
    return m, before


# ---- (a) the five lit cases: lo=0, hi=%arg1, step 1 (or 10), compare %iv <pred> %mid -------------------
# Expected structure, read off the CHECK lines of loop-split.mlir:
#   sgt  (:3-32)    no addi; loop 1 runs the else-branch (subf), loop 2 the then-branch (addf)
#   sge  (:36-66)   mid + (-1); loop 1 subf, loop 2 addf
#   slt  (:70-97)   loop 1 addf, loop 2 subf
#   sle  (:101-131) mid + 1;   loop 1 addf, loop 2 subf
#   step10 (:135-167) slt, step 10: loop 1 addf up to a rounded mid, loop 2 subf from the same mid
LIT = [
    ("sgt", 1, 0, P.TXIR_FOLDED_FALSE, P.TXIR_FOLDED_TRUE),
    ("sge", 1, -1, P.TXIR_FOLDED_FALSE, P.TXIR_FOLDED_TRUE),
    ("slt", 1, 0, P.TXIR_FOLDED_TRUE, P.TXIR_FOLDED_FALSE),
    ("sle", 1, +1, P.TXIR_FOLDED_TRUE, P.TXIR_FOLDED_FALSE),
]


@pytest.mark.parametrize("pred,step,adjust,fold1,fold2", LIT)
def test_lit_known_answers_as_written(built_libs, pred, step, adjust, fold1, fold2):
    hi, mid = 1000, 417
    m, _ = run_pass(P.make_loop(0, hi, step, pred, mid), "as-written")
    loops = m.loops()
    assert len(loops) == 2
    assert (loops[0]["lo"], loops[0]["hi"]) == (0, mid + adjust)
    assert (loops[1]["lo"], loops[1]["hi"]) == (mid + adjust, hi)
    assert loops[0]["fold"] == fold1 and loops[1]["fold"] == fold2
    assert loops[1]["origin"] == 0 and loops[0]["origin"] == -1


def test_lit_step10_structure(built_libs):
    for mode in ("as-written", "intent"):
        m, _ = run_pass(P.make_loop(0, 1000, 10, "slt", 417), mode)
        a, b = m.loops()
        assert a["step"] == b["step"] == 10
        assert a["fold"] == P.TXIR_FOLDED_TRUE and b["fold"] == P.TXIR_FOLDED_FALSE  # addf then subf
        assert a["hi"] == b["lo"] and a["hi"] % 10 == 0 and a["hi"] >= 417              # "mid-point is rounded up"
    # intent: the smallest grid point >= 417
    m, before = run_pass(P.make_loop(0, 1000, 10, "slt", 417), "intent")
    assert m.loops()[0]["hi"] == 420 and m.simulate(0) == before


# ---- (b) as-written mode equals the C restatement of LoopSplit.cpp on a sweep ----------------------------
def test_as_written_matches_oracle(built_libs, oracle):
    rng = random.Random(7)
    cases = []
    for pred, step, ivop in itertools.product(ORACLE_PRED, (1, 2, 10, 128), (0, 1)):
        for _ in range(6):
            lo = rng.choice([0, 0, 3, -20, 128])
            cases.append((lo, lo + rng.randrange(0, 3000), step, pred, ivop, rng.randrange(-50, 3100)))
    cases += [(0, 4160, 128, "slt", 0, 4096), (0, 16384, 128, "sge", 0, 8192), (0, 100, 1, "sge", 0, -2**31)]
    for lo, hi, step, pred, ivop, v in cases:
        r = LsResult()
        oracle.ls_bisect_as_written(lo, hi, step, 1, ORACLE_PRED[pred], ivop, v, 1, ctypes.byref(r))
        m, _ = run_pass(P.make_loop(lo, hi, step, pred, v, iv_operand=ivop), "as-written")
        loops = m.loops()
        assert r.split == 1 and len(loops) == 2, (lo, hi, step, pred, ivop, v)
        assert loops[0]["hi"] == r.mid and loops[1]["lo"] == r.mid, (lo, hi, step, pred, ivop, v)
        assert loops[0]["fold"] == (P.TXIR_FOLDED_TRUE if r.cmp1 else P.TXIR_FOLDED_FALSE)
        assert loops[1]["fold"] == (P.TXIR_FOLDED_TRUE if r.cmp2 else P.TXIR_FOLDED_FALSE)


def test_rejections_match_oracle(built_libs, oracle):
    """Non-constant step, non-positive step, loop-variant comparand, unsupported predicate: no split
    (LoopSplit.cpp:128-138, :107-123, :57-59)."""
    variants = [
        dict(step_is_constant=False), dict(invariant=False),
    ]
    for kw in variants:
        for mode in ("as-written", "intent"):
            m, _ = run_pass(P.make_loop(0, 100, 1, "slt", 50, **kw), mode)
            assert len(m.loops()) == 1
        r = LsResult()
        oracle.ls_bisect_as_written(0, 100, 1, int(kw.get("step_is_constant", True)), 0, 0, 50,
                                    int(kw.get("invariant", True)), ctypes.byref(r))
        assert r.split == 0
    for step in (0, -1):
        m, _ = run_pass(P.make_loop(0, 100, step, "slt", 50), "intent")
        assert len(m.loops()) == 1
    for pred in ("eq", "ne"):
        m, _ = run_pass(P.make_loop(0, 100, 1, pred, 50), "intent")
        assert len(m.loops()) == 1
    loop = P.make_loop(0, 100, 1, "slt", 50)
    loop.has_cmp = 0
    m, _ = run_pass(loop, "intent")
    assert len(m.loops()) == 1


# ---- (c) intent mode keeps the meaning of every loop; as-written mode is known not to --------------------
def test_intent_mode_preserves_semantics(built_libs, oracle):
    rng = random.Random(11)
    for pred, step, ivop in itertools.product(ORACLE_PRED, (1, 3, 10, 64), (0, 1)):
        for _ in range(8):
            lo = rng.choice([0, 0, 5, 64])
            hi = lo + rng.randrange(0, 700)
            v = rng.randrange(-30, 800)
            loop = P.make_loop(lo, hi, step, pred, v, iv_operand=ivop)
            m, before = run_pass(loop, "intent")
            assert before == oracle.ls_run_original(lo, hi, step, ORACLE_PRED[pred], ivop, v)
            assert m.simulate(0) == before, (lo, hi, step, pred, ivop, v, str(m))
            loops = m.loops()
            assert lo <= loops[0]["hi"] <= max(hi, lo)
            assert all(l["fold"] != P.TXIR_NOT_FOLDED for l in loops)


def test_as_written_quirks_are_reproduced(built_libs):
    # `iv > V` with step 1 splits at V, one iteration early (the iteration iv == V lands in loop 2
    # with the compare folded to true although V > V is false).
    m, before = run_pass(P.make_loop(0, 100, 1, "sgt", 37), "as-written")
    assert m.loops()[0]["hi"] == 37 and m.simulate(0) != before
    # `iv < V` with an aligned V and step != 1 is pushed a full step too far.
    m, before = run_pass(P.make_loop(0, 4160, 128, "slt", 4096), "as-written")
    assert m.loops()[0]["hi"] == 4096 + 128 and m.simulate(0) != before
    # `iv >= V` with an aligned V and step != 1: the two adjustments cancel (the attention use-case).
    m, before = run_pass(P.make_loop(0, 1024, 64, "sge", 512), "as-written")
    assert m.loops()[0]["hi"] == 512 and m.simulate(0) == before


def test_pass_is_idempotent_and_keeps_other_loops(built_libs):
    P.load_default_plugins()
    m = P.Module()
    m.add_loop(P.make_loop(0, 10, 1, "eq", 5))          # untouched
    m.add_loop(P.make_loop(0, 100, 1, "slt", 40))        # split
    pm = P.PassManager()
    pm.add("loop_split")
    pm.add("loop_split")                                  # second run finds only folded compares
    assert pm.run(m) == 0
    loops = m.loops()
    assert [(l["lo"], l["hi"]) for l in loops] == [(0, 10), (0, 40), (40, 100)]
    assert loops[2]["origin"] == 1


# ---- the tt.dot K loop ------------------------------------------------------------------------------------
def test_dot_k_loop_split_point(built_libs):
    import torch
    from triton_ext_b200 import backend as B
    pr = B.make_problem(4096, 4096, 4160, torch.bfloat16, torch.bfloat16)
    cfg, info, m = P.lower_dot(pr, 128)
    loops = m.loops()
    assert [(l["lo"], l["hi"], l["step"]) for l in loops] == [(0, 4096, 128), (4096, 4160, 128)]
    assert loops[0]["fold"] == P.TXIR_FOLDED_TRUE and loops[1]["fold"] == P.TXIR_FOLDED_FALSE
    assert cfg.k_split_point == 4096
    assert info["k_main_iters"] * info["block_k"] == 4096 and info["k_tail_iters"] == 1 and info["k_tail_mmas"] == 4
    # K a multiple of BLOCK_K: no remainder loop work
    cfg, info, m = P.lower_dot(B.make_problem(512, 512, 512, torch.float16, torch.float16), 32)
    assert cfg.k_split_point == 512 and info["k_tail_iters"] == 0
    # K smaller than BLOCK_K: everything is remainder
    cfg, info, m = P.lower_dot(B.make_problem(256, 256, 40, torch.bfloat16, torch.bfloat16), 64)
    assert cfg.k_split_point == -1 and info["k_main_iters"] == 0 and info["k_tail_iters"] == 1
    assert info["k_tail_mmas"] == 3  # ceil(40 / 16)


def test_dot_as_written_split_is_rejected_by_the_backend(built_libs):
    """As written, the reference's arithmetic moves `k < K_main` one step too far when K_main is aligned,
    which would run the partial block unmasked; the backend pass refuses such a split."""
    import torch
    from triton_ext_b200 import backend as B
    pr = B.make_problem(4096, 4096, 4160, torch.bfloat16, torch.bfloat16)
    with pytest.raises(RuntimeError, match="unmasked"):
        P.lower_dot(pr, 128, attrs={"loop_split.mode": "as-written"})


@pytest.mark.parametrize("mode", ["intent", "as-written"])
def test_attention_kv_loop_split_is_what_the_kernel_runs(built_libs, mode):
    """The reference's use case (06-fused-attention.py:59-64): `for start_n in range(0, hi, BLOCK_N)` with
    `start_n >= causal_start`, causal_start = start_m * BLOCK_M. sge with a step > 1 and an aligned comparand is
    the one predicate for which the reference's arithmetic and its intent agree (-step, then +step), so both modes
    must give the off-band / on-band loops the attention kernel executes per 128-row sub-tile."""
    from triton_ext_b200 import attention as A
    block = 128
    for n_ctx, start_m in [(1024, 0), (1024, 3), (1024, 7), (4096, 17), (384, 2)]:
        causal_start = start_m * block
        hi = (start_m + 1) * block          # the kernel does not visit the fully masked blocks above the diagonal
        loop = P.make_loop(0, hi, block, "sge", causal_start)
        m, before = run_pass(loop, mode)
        loops = m.loops()
        n, unmasked = A.kv_loop_split(n_ctx, causal_start, True, block)
        assert (n, unmasked) == (start_m + 1, start_m)
        if start_m == 0:
            # nothing below the diagonal: the off-band loop is empty
            live = [l for l in loops if l["hi"] > l["lo"]]
            assert [(l["lo"], l["hi"]) for l in live] == [(0, block)]
            assert live[0]["fold"] in (P.TXIR_FOLDED_TRUE, P.TXIR_NOT_FOLDED)
        else:
            assert [(l["lo"], l["hi"], l["step"]) for l in loops] == [(0, unmasked * block, block), (unmasked * block, n * block, block)]
            assert loops[0]["fold"] == P.TXIR_FOLDED_FALSE and loops[1]["fold"] == P.TXIR_FOLDED_TRUE
        assert m.simulate(0) == before      # same result as the unsplit loop

