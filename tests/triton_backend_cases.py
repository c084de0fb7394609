"""The Triton backend entry point on CPU: TTIR of @triton.jit K loops -> proof -> bound GEMM -> pass pipeline.

Nothing here needs a GPU: Triton's front end, the analysis, triton.compile() through the backend, and a
whole `kernel[grid](...)` launch under a driver whose launcher stops before the CUDA call. Run by
test_triton_backend.py in a process of its own (Triton must not be in interpreter mode here).
"""
import math

import pytest
import torch

triton = pytest.importorskip("triton")

import jit_kernels as jk  # noqa: E402
from triton_ext_b200 import triton_backend as tbk  # noqa: E402
from triton_ext_b200.triton_backend import compiler, driver, ttir  # noqa: E402

PTR = {"bf16": "*bf16", "f16": "*fp16", "f8e4m3": "*fp8e4nv"}


def split_sig(dt="bf16", out="bf16", ones=("stride_ak", "stride_bn", "stride_cn"), bm=128, bn=128, bk=128):
    sig = {"a_ptr": PTR[dt], "b_ptr": PTR[dt], "c_ptr": PTR[out], "M": "i32", "N": "i32", "K": "i32"}
    cx = {}
    for s in ("stride_am", "stride_ak", "stride_bk", "stride_bn", "stride_cm", "stride_cn"):
        sig[s] = "constexpr" if s in ones else "i32"
        if s in ones:
            cx[s] = 1
    sig.update({"K_MAIN": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"})
    cx.update({"BLOCK_M": bm, "BLOCK_N": bn, "BLOCK_K": bk})
    return sig, cx


def small_sig(dt="bf16"):
    sig = {"a_ptr": PTR[dt], "b_ptr": PTR[dt], "c_ptr": PTR[dt], "K": "i32", "stride_am": "i32", "stride_bk": "i32",
           "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    return sig, {"BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_K": 32}


def grouped_sig(bm=64, bn=128, bk=32, group=4):
    sig = {"a_ptr": "*fp16", "b_ptr": "*fp16", "c_ptr": "*fp16", "M": "i32", "N": "i32", "K": "i32", "stride_am": "i32",
           "stride_ak": "constexpr", "stride_bk": "constexpr", "stride_bn": "i32", "stride_cm": "i32",
           "stride_cn": "constexpr", "alpha": "fp32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr",
           "BLOCK_K": "constexpr", "GROUP": "constexpr"}
    cx = {"stride_ak": 1, "stride_bk": 1, "stride_cn": 1, "BLOCK_M": bm, "BLOCK_N": bn, "BLOCK_K": bk, "GROUP": group}
    return sig, cx


def test_ttir_has_the_loop_split_shape():
    """The IR the analysis reads is the one LoopSplit rewrites: scf.for + cmpi slt on the IV + scf.if."""
    text = ttir.strip_locations(compiler.lower_to_ttir(jk.split_kloop, *split_sig()))
    assert "scf.for" in text and "tt.dot" in text and "scf.if" in text
    assert any("arith.cmpi slt" in l and "%K_MAIN" in l for l in text.splitlines())


def test_split_kloop_match():
    m = compiler.analyse(jk.split_kloop, *split_sig(), split=False)
    assert (m.a_arg, m.b_arg, m.c_arg) == ("a_ptr", "b_ptr", "c_ptr")
    assert (m.block_m, m.block_n, m.block_k) == (128, 128, 128)
    assert (m.ab_dtype, m.out_dtype) == ("bf16", "bf16")
    assert (m.a_row_stride, m.a_k_stride, m.b_k_stride, m.b_col_stride) == ("stride_am", "1", "stride_bk", "1")
    assert (m.row0, m.col0) == ("128*pid_x", "128*pid_y")
    assert (m.loop_lo, m.loop_hi, m.loop_step, m.k_per_iv) == ("0", "K", 128, 1)
    assert (m.k_bound, m.split_pred, m.split_comparand) == ("K", "slt", "K_MAIN")
    assert m.alpha is None
    assert ttir.DotKernelMatch.from_json(m.to_json()) == m


def test_loop_split_on_the_kernels_own_ir():
    """LoopSplit as a rewrite of the real IR: two scf.for where there was one, the compare gone, unmasked loads
    only in the first and masked loads only in the second (after Triton's canonicaliser), accepted by Triton's
    MLIR parser; and the matcher reads the pair back as one loop split at the mid point."""
    from triton_ext_b200.triton_backend import loop_split_ir

    sig, cx = split_sig()
    before = ttir.strip_locations(compiler.lower_to_ttir(jk.split_kloop, sig, cx))
    assert before.count("scf.for") == 1 and before.count("scf.if") == 1
    raw, n = loop_split_ir.split_loops(before)
    assert n == 1 and raw.count("scf.for") == 2 and "arith.constant true" in raw and "arith.constant false" in raw
    names: list = []
    after = ttir.strip_locations(compiler.lower_to_ttir(jk.split_kloop, sig, cx, split=True, arg_names_out=names))
    assert names[:3] == ["a_ptr", "b_ptr", "c_ptr"] and names[-1] == "K_MAIN"
    assert after.count("scf.for") == 2 and "scf.if" not in after
    first, second = after.split("scf.for")[1:]
    assert "tt.load" in first and "arith.cmpi" not in first       # main loop: no compare, no mask
    assert second.count("arith.cmpi slt") == 2                      # remainder loop: the two K masks
    assert "arith.ceildivsi" in after and "arith.minsi" in after    # the mid point
    m = ttir.match_dot_kernel(after, names)
    assert (m.loop_lo, m.loop_hi, m.split_pred) == ("0", "K", "slt")
    assert m.split_comparand == "Min(128*ceiling(Max(0, K_MAIN)/128), Max(0, K))"
    s = dict(M=1024, N=512, K=4160, stride_am=4160, stride_bk=512, stride_cm=512)
    assert ttir.bind(m, dict(s, K_MAIN=4096), (8, 4)).k_main == 4096
    assert ttir.bind(m, dict(s, K_MAIN=1000), (8, 4)).k_main == 1024   # mid rounds up to the step
    assert ttir.bind(m, dict(s, K_MAIN=0), (8, 4)).k_main == 0
    with pytest.raises(ttir.NotCanonical, match="unmasked load run past"):
        ttir.bind(m, dict(s, K_MAIN=4160), (8, 4))
    # a loop without a compare on its induction variable is left alone
    plain = ttir.strip_locations(compiler.lower_to_ttir(jk.plain_kloop, *plain_sig()))
    assert loop_split_ir.split_loops(plain)[1] == 0


def test_loop_split_peels_the_remainder_of_an_always_masked_k_loop():
    """What the reference leaves open (LoopSplit.cpp:105, "TODO: add support for mask logic"): a K loop whose loads
    are masked by `k + arange(BLOCK_K) < K` in every iteration has no scalar compare to split on, but its masks are
    all-true while k + BLOCK_K <= K. The rewrite splits there, the first loop loses its K masks (Triton's canonicaliser
    folds a constant-true mask away) and keeps the row / column masks, the second is the masked remainder."""
    from triton_ext_b200.triton_backend import loop_split_ir

    sig = {"a_ptr": "*bf16", "bt_ptr": "*bf16", "c_ptr": "*bf16", "M": "i32", "N": "i32", "K": "i32", "stride_am": "i32",
           "stride_bn": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    cx = {"BLOCK_M": 128, "BLOCK_N": 64, "BLOCK_K": 64}
    before = ttir.strip_locations(compiler.lower_to_ttir(jk.nt_kloop, sig, cx))
    assert before.count("scf.for") == 1 and "scf.if" not in before
    raw, n = loop_split_ir.split_loops(before)
    assert n == 1 and raw.count("arith.constant dense<true> : tensor<1x64xi1>") >= 1
    assert loop_split_ir.split_loops(before, mode="as-written")[1] == 0      # the reference's pass does not split it
    names: list = []
    after = ttir.strip_locations(compiler.lower_to_ttir(jk.nt_kloop, sig, cx, split=True, arg_names_out=names))
    main, rest = after.split("scf.for")[1:]
    k_mask = lambda body: sum(1 for l in body.split("scf.yield")[0].splitlines() if "arith.cmpi slt" in l and "1x64" in l)
    assert k_mask(main) == 0 and k_mask(rest) >= 1
    assert main.count("tt.load") == 2 and rest.split("scf.yield")[0].count("tt.load") == 2
    m = ttir.match_dot_kernel(after, names)
    assert m.split_comparand == "Min(64*ceiling(Max(0, K - 63)/64), Max(0, K))" and m.k_bound == "K"
    for K in list(range(1, 200)) + [500, 512, 4096, 4160]:
        b = ttir.bind(m, dict(M=300, N=200, K=K, stride_am=4224, stride_bn=4224, stride_cm=256), (3, 4))
        assert (b.k, b.k_main) == (K, (K // 64) * 64), K


LIT_CASE = """
module {
  tt.func public @lit(%out: !tt.ptr<i32>, %n: i32, %c: i32) {
    %c0 = arith.constant 0 : i32
    %c1 = arith.constant 1 : i32
    %cS = arith.constant STEP : i32
    %r = scf.for %i = %c0 to %n step %cS iter_args(%acc = %c0) -> (i32)  : i32 {
      %p = arith.cmpi PRED, LHS, RHS : i32
      %v = arith.addi %i, %c1 : i32
      %a = arith.addi %acc, %v : i32
      %s = arith.subi %acc, %v : i32
      %x = arith.select %p, %a, %s : i32
      scf.yield %x : i32
    }
    tt.store %out, %r : !tt.ptr<i32>
    tt.return
  }
}
"""


@pytest.mark.parametrize("pred,swap,step", [("slt", False, 1), ("sle", False, 1), ("sgt", False, 1), ("sge", False, 1),
                                            ("slt", False, 10), ("sgt", True, 3), ("sle", True, 7)])
def test_loop_split_ir_keeps_the_meaning_of_the_lit_test_loops(pred, swap, step):
    """The loops of the reference's lit test (pass/LoopSplit/test/loop-split.mlir: acc +/- (iv + 1) selected by a
    compare of the induction variable; sgt / sge / slt / sle and a step-10 case), bisected on the IR text and
    executed before and after by a tiny interpreter over every small bound and comparand."""
    from triton_ext_b200.triton_backend import loop_split_ir

    text = (LIT_CASE.replace("STEP", str(step)).replace("PRED", pred)
            .replace("LHS", "%c" if swap else "%i").replace("RHS", "%i" if swap else "%c"))
    new, n = loop_split_ir.split_loops(text)
    assert n == 1 and new.count("scf.for") == 2
    for bound in range(0, 24, 5):
        for comparand in range(-3, 27, 2):
            assert run_scalar_ir(new, bound, comparand) == run_scalar_ir(text, bound, comparand), (bound, comparand)


def run_scalar_ir(text: str, n: int, c: int) -> int:
    """Execute the scalar i32 subset the lit loops use (constants, addi, subi, muli, maxsi, minsi, ceildivsi, cmpi,
    select, scf.for with one iter_arg) and return the stored value."""
    _, _, ops = ttir.parse_module(text)
    u = lambda v: v & 0xFFFFFFFF      # an i32 read as unsigned
    cmp = {"slt": lambda a, b: a < b, "sle": lambda a, b: a <= b, "sgt": lambda a, b: a > b, "sge": lambda a, b: a >= b,
           "ult": lambda a, b: u(a) < u(b), "ule": lambda a, b: u(a) <= u(b), "ugt": lambda a, b: u(a) > u(b),
           "uge": lambda a, b: u(a) >= u(b)}
    arith = {"arith.addi": lambda a, b: a + b, "arith.subi": lambda a, b: a - b, "arith.muli": lambda a, b: a * b,
             "arith.maxsi": max, "arith.minsi": min, "arith.ceildivsi": lambda a, b: -((-a) // b),
             "arith.remui": lambda a, b: a % b}

    def run(block, env):
        for op in block:
            g = lambda k: env[op.operands[k]]
            if op.name == "arith.constant":
                tok = op.rest.split(" :")[0].strip()
                env[op.results[0]] = {"true": True, "false": False}.get(tok, None if tok in ("true", "false") else tok)
                if not isinstance(env[op.results[0]], bool):
                    env[op.results[0]] = int(tok)
            elif op.name in arith:
                env[op.results[0]] = arith[op.name](g(0), g(1))
            elif op.name == "arith.cmpi":
                env[op.results[0]] = cmp[op.rest.split(",")[0].strip()](g(0), g(1))
            elif op.name == "arith.select":
                env[op.results[0]] = g(1) if g(0) else g(2)
            elif op.name == "scf.for":
                lo, hi, st = (env[o] for o in op.operands)
                (name, init), = op.extra["iters"]
                acc = env[init]
                for i in range(lo, hi, st):
                    inner = dict(env)
                    inner[op.extra["iv"]] = i
                    inner[name] = acc
                    acc = run(op.regions[0], inner)
                env[op.results[0]] = acc
            elif op.name == "scf.yield":
                return g(0)
            elif op.name == "tt.store":
                env["stored"] = g(1)
        return None

    env = {"%out": None, "%n": n, "%c": c}
    run(ops, env)
    return env["stored"]


def plain_sig():
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*fp32", "K": "i32", "stride_am": "i32", "stride_ak": "constexpr",
           "stride_bk": "i32", "stride_bn": "constexpr", "stride_cm": "i32", "BLOCK_M": "constexpr",
           "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    return sig, {"stride_ak": 1, "stride_bn": 1, "BLOCK_M": 128, "BLOCK_N": 64, "BLOCK_K": 64}


def test_split_kloop_bind_benchmark_shape():
    """The 8192 x 8192 x 4160 bf16 case: 32 full K blocks of 128 and a 64-wide remainder."""
    m = compiler.analyse(jk.split_kloop, *split_sig())
    s = dict(M=8192, N=8192, K=4160, stride_am=4160, stride_bk=8192, stride_cm=8192, K_MAIN=4096)
    b = ttir.bind(m, s, (64, 64))
    assert (b.m, b.n, b.k, b.a_layout, b.b_layout, b.lda, b.ldb, b.ldc) == (8192, 8192, 4160, "row", "row", 4160, 8192, 8192)
    assert (b.block_k, b.k_main, b.alpha) == (128, 4096, 1.0)
    # an earlier split point is still right (more iterations masked), a later one would read past K unmasked
    assert ttir.bind(m, dict(s, K_MAIN=2048), (64, 64)).k_main == 2048
    with pytest.raises(ttir.NotCanonical, match="unmasked load run past"):
        ttir.bind(m, dict(s, K_MAIN=4160), (64, 64))
    # this kernel has no row or column masks: the grid alone says how much of C is computed
    assert ttir.bind(m, s, (64, 63)).n == 63 * 128
    with pytest.raises(ttir.NotCanonical, match="does not cover"):
        ttir.bind(m, s, (64, 64, 2))


def test_transposed_operands_bind_as_column_major():
    sig, cx = split_sig("f16", "f16", ones=("stride_am", "stride_bk", "stride_cn"))
    m = compiler.analyse(jk.split_kloop, sig, cx)
    b = ttir.bind(m, dict(M=256, N=384, K=200, stride_ak=256, stride_bn=200, stride_cm=384, K_MAIN=128), (2, 3))
    assert (b.a_layout, b.lda, b.b_layout, b.ldb, b.k_main) == ("col", 256, "col", 200, 128)
    sig, cx = split_sig("f16", "f16", ones=("stride_cn",))
    m = compiler.analyse(jk.split_kloop, sig, cx)
    with pytest.raises(ttir.NotCanonical, match="no unit stride"):
        ttir.bind(m, dict(M=256, N=384, K=200, stride_am=400, stride_ak=2, stride_bk=384, stride_bn=1, stride_cm=384,
                          K_MAIN=128), (2, 3))


def test_column_major_output_exchanges_the_operands():
    sig, cx = split_sig("f16", "f16", ones=("stride_ak", "stride_bn", "stride_cm"))
    m = compiler.analyse(jk.split_kloop, sig, cx)
    b = ttir.bind(m, dict(M=256, N=384, K=200, stride_am=208, stride_bk=384, stride_cn=256, K_MAIN=128), (2, 3))
    # C^T [384, 256] = B^T [384, 200] (column-major view of the row-major B) @ A^T [200, 256]
    assert b.swapped and (b.m, b.n, b.k) == (384, 256, 200)
    assert (b.a_layout, b.lda, b.b_layout, b.ldb, b.ldc) == ("col", 384, "col", 208, 256)
    with pytest.raises(ttir.NotCanonical, match="no unit stride"):
        sig2, cx2 = split_sig("f16", "f16", ones=("stride_ak", "stride_bn"))
        ttir.bind(compiler.analyse(jk.split_kloop, sig2, cx2),
                  dict(M=256, N=384, K=200, stride_am=208, stride_bk=384, stride_cm=2, stride_cn=512, K_MAIN=128), (2, 3))


def test_grouped_masked_kloop():
    """Block-counting loop, pointers carried by the loop, a swizzled 1-D grid, three-way masks, a scalar scale."""
    m = compiler.analyse(jk.grouped_masked_kloop, *grouped_sig())
    assert (m.loop_step, m.k_per_iv, m.block_k) == (1, 32, 32)
    assert (m.k_bound, m.m_bound, m.n_bound, m.alpha) == ("K", "M", "N", "alpha")
    # LoopSplit peels this loop's masked remainder; without that stage the kernel reads as one unsplit loop
    assert m.split_pred == "slt" and m.split_is_loop_bound
    assert compiler.analyse(jk.grouped_masked_kloop, *grouped_sig(), split=False).split_pred is None
    for M, N, K in ((1000, 300, 1111), (64, 128, 32), (65, 129, 33), (4096, 4096, 64)):
        grid = (math.ceil(M / 64) * math.ceil(N / 128),)
        s = dict(M=M, N=N, K=K, stride_am=K, stride_bn=K, stride_cm=N)
        b = ttir.bind(m, s, grid, {"alpha": 0.5})
        assert (b.m, b.n, b.k, b.a_layout, b.b_layout, b.alpha) == (M, N, K, "row", "col", 0.5)
        assert b.k_main == (K // 32) * 32
        if grid[0] > 1:
            with pytest.raises(ttir.NotCanonical, match="does not cover"):
                ttir.bind(m, s, (grid[0] - 1,), {"alpha": 0.5})


def test_plain_kloop_without_masks():
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*fp32", "K": "i32", "stride_am": "i32", "stride_ak": "constexpr",
           "stride_bk": "i32", "stride_bn": "constexpr", "stride_cm": "i32", "BLOCK_M": "constexpr",
           "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    m = compiler.analyse(jk.plain_kloop, sig, {"stride_ak": 1, "stride_bn": 1, "BLOCK_M": 128, "BLOCK_N": 64, "BLOCK_K": 64})
    assert (m.k_bound, m.m_bound, m.n_bound, m.out_dtype) == (None, None, None, "f32")
    assert (m.row0, m.col0) == ("128*pid_y", "64*pid_x")
    b = ttir.bind(m, dict(K=512, stride_am=512, stride_bk=320, stride_cm=320), (5, 3))
    assert (b.m, b.n, b.k, b.k_main) == (384, 320, 512, 512)


def test_loop_split_peels_a_block_counting_loop_with_carried_pointers():
    """The other common form: the loop counts K blocks, the pointers are carried by the loop, the masks compare
    arange(BLOCK_K) with `K - kb * BLOCK_K`. Split where kb * BLOCK_K + BLOCK_K <= K stops holding; the second loop
    starts from the pointers the first one leaves behind."""
    sig, cx = split_sig("f16", "f16", bm=128, bn=64, bk=64)
    del sig["K_MAIN"]
    names: list = []
    after = ttir.strip_locations(compiler.lower_to_ttir(jk.wrapped_kloop, sig, cx, split=True, arg_names_out=names))
    assert after.count("scf.for") == 2 and "arith.floordivsi" in after or "arith.divsi" in after
    main, rest = after.split("scf.for")[1:]
    assert "arith.cmpi" not in main.split("scf.yield")[0] and "arith.cmpi slt" in rest.split("scf.yield")[0]
    m = ttir.match_dot_kernel(after, names)
    assert m.split_is_loop_bound and (m.loop_step, m.k_per_iv) == (1, 64)
    for K in (1, 63, 64, 65, 500, 4160):
        b = ttir.bind(m, dict(M=300, N=200, K=K, stride_am=4224, stride_bk=200, stride_cm=200), (3 * 4,))
        assert (b.k, b.k_main) == (K, (K // 64) * 64), K


def test_wrapped_indices_need_a_masked_store():
    """Loads whose row / column indices are taken modulo M / N (no row or column masks in the loop) are the
    plain GEMM as long as the store masks with the same bounds."""
    sig, cx = split_sig("f16", "f16", bm=128, bn=64, bk=64)
    del sig["K_MAIN"]
    m = compiler.analyse(jk.wrapped_kloop, sig, cx)
    assert (m.k_bound, m.m_bound, m.n_bound, m.k_per_iv, m.loop_step) == ("K", "M", "N", 64, 1)
    b = ttir.bind(m, dict(M=300, N=200, K=500, stride_am=500, stride_bk=200, stride_cm=200), (3 * 4,))
    assert (b.m, b.n, b.k, b.k_main) == (300, 200, 500, 448)
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16", "M": "i32", "K": "i32", "stride_am": "i32",
           "stride_bk": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    with pytest.raises(ttir.NotCanonical, match="wrapped by something that is not the bound the store masks with"):
        compiler.analyse(jk.wrapped_unmasked_store_kloop, sig, {"BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_K": 32})


def test_persistent_kernel_with_a_tile_loop():
    """A loop over tiles around the K loop, a helper function (inlined) for the tile order: the origin becomes a
    function of the tile loop's induction variable and bind() walks every program's iterations."""
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16", "M": "i32", "N": "i32", "K": "i32", "stride_am": "i32",
           "stride_bk": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr",
           "BLOCK_K": "constexpr", "GROUP": "constexpr"}
    m = compiler.analyse(jk.persistent_kloop, sig, {"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 64, "GROUP": 8})
    assert m.tile_loop == ["pid_x", "floor(M/128 + 127/128)*floor(N/128 + 127/128)", "nprog_x"]
    assert "tile_iv" in m.row0 and "tile_iv" in m.col0 and "pid_x" not in m.row0
    assert ttir.DotKernelMatch.from_json(m.to_json()) == m
    s = dict(M=3000, N=2000, K=500, stride_am=512, stride_bk=2048, stride_cm=2048)
    for programs in (148, 7, 1, 1000):
        b = ttir.bind(m, s, (programs,))
        assert (b.m, b.n, b.k, b.k_main) == (3000, 2000, 500, 448)
    with pytest.raises(ttir.NotCanonical, match="does not cover"):
        ttir.bind(m, s, (4, 2))  # programs of the second grid row repeat the tiles of the first


def test_packaged_kernel_keeps_row_and_column_masks_under_the_split():
    """kernels.dot_kloop: the side of the split without a K mask still masks rows and columns."""
    from triton_ext_b200.triton_backend import kernels

    m = compiler.analyse(kernels.dot_kloop, *split_sig(), split=False)
    assert (m.k_bound, m.m_bound, m.n_bound, m.split_pred, m.split_comparand) == ("K", "M", "N", "slt", "K_MAIN")
    m = compiler.analyse(kernels.dot_kloop, *split_sig())  # the same after LoopSplit has made two loops of it
    assert (m.k_bound, m.m_bound, m.n_bound, m.split_pred) == ("K", "M", "N", "slt")
    assert m.split_comparand == "Min(128*ceiling(Max(0, K_MAIN)/128), Max(0, K))"
    b = ttir.bind(m, dict(M=4096, N=4096, K=4160, stride_am=4160, stride_bk=4096, stride_cm=4096, K_MAIN=4096), (32, 32))
    assert (b.m, b.n, b.k, b.k_main) == (4096, 4096, 4160, 4096)


def test_transposed_tile_in_registers():
    """tl.trans of the loaded B tile (B stored [N, K]) binds as a column-major B."""
    sig = {"a_ptr": "*bf16", "bt_ptr": "*bf16", "c_ptr": "*bf16", "M": "i32", "N": "i32", "K": "i32", "stride_am": "i32",
           "stride_bn": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    m = compiler.analyse(jk.nt_kloop, sig, {"BLOCK_M": 128, "BLOCK_N": 64, "BLOCK_K": 64})
    assert (m.b_arg, m.b_k_stride, m.b_col_stride, m.block_n, m.block_k) == ("bt_ptr", "1", "stride_bn", 64, 64)
    b = ttir.bind(m, dict(M=300, N=200, K=500, stride_am=512, stride_bn=512, stride_cm=256), (3, 4))
    assert (b.b_layout, b.ldb, b.m, b.n, b.k) == ("col", 512, 300, 200, 500)


def test_block_pointer_kernel():
    """tl.make_block_ptr / tl.advance with boundary checks (how the reference's attention addresses its operands,
    06-fused-attention.py:180-215): Triton rewrites them to pointer arithmetic on loop-carried i64 offsets and
    two-sided masks; the `index >= 0` halves are trivially true."""
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16", "M": "i32", "N": "i32", "K": "i32", "stride_am": "i32",
           "stride_bk": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    m = compiler.analyse(jk.block_pointer_kloop, sig, {"BLOCK_M": 128, "BLOCK_N": 64, "BLOCK_K": 64})
    assert (m.k_bound, m.m_bound, m.n_bound, m.row0, m.col0) == ("K", "M", "N", "128*pid_x", "64*pid_y")
    b = ttir.bind(m, dict(M=300, N=200, K=500, stride_am=512, stride_bk=256, stride_cm=256), (3, 4))
    assert (b.m, b.n, b.k, b.k_main) == (300, 200, 500, 448)


def test_single_dot_without_a_loop():
    sig = {"a_ptr": "*fp8e5", "b_ptr": "*fp8e5", "c_ptr": "*fp16", "M": "i32", "N": "i32", "K": "i32", "stride_am": "i32",
           "stride_bk": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    m = compiler.analyse(jk.single_dot, sig, {"BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_K": 128})
    assert (m.ab_dtype, m.out_dtype, m.loop_lo, m.loop_hi, m.loop_step, m.k_bound) == ("f8e5m2", "f16", "0", "128", 128, "K")
    b = ttir.bind(m, dict(M=100, N=70, K=96, stride_am=96, stride_bk=80, stride_cm=80), (2, 2))
    assert (b.m, b.n, b.k, b.k_main) == (100, 70, 96, 0)
    with pytest.raises(ttir.NotCanonical, match="covers 128 of K=200"):
        ttir.bind(m, dict(M=100, N=70, K=200, stride_am=208, stride_bk=80, stride_cm=80), (2, 2))


def test_tensor_descriptor_kernel():
    """tl.make_tensor_descriptor / desc.load / desc.store (the form of the reference's _attn_fwd_tma,
    06-fused-attention.py:94-139): the bounds are the descriptor shapes, the fill is zero."""
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16", "M": "i32", "N": "i32", "K": "i32", "stride_am": "i32",
           "stride_bk": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    m = compiler.analyse(jk.descriptor_kloop, sig, {"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 64})
    assert (m.k_bound, m.m_bound, m.n_bound) == ("K", "M", "N")
    assert (m.a_row_stride, m.a_k_stride, m.b_k_stride, m.b_col_stride, m.c_row_stride) == \
        ("stride_am", "1", "stride_bk", "1", "stride_cm")
    b = ttir.bind(m, dict(M=300, N=200, K=500, stride_am=512, stride_bk=256, stride_cm=256), (3, 2))
    assert (b.m, b.n, b.k, b.k_main, b.lda, b.ldb, b.ldc) == (300, 200, 500, 448, 512, 256, 256)


def scaled_sig(dt="f8e4m3"):
    sig = {"a_ptr": PTR[dt], "b_ptr": PTR[dt], "c_ptr": "*bf16", "rs_ptr": "*fp32", "cs_ptr": "*fp32", "M": "i32",
           "N": "i32", "K": "i32", "stride_am": "i32", "stride_bk": "i32", "stride_cm": "i32", "alpha": "fp32",
           "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    return sig, {"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 128}


@pytest.mark.parametrize("dt", ["f8e4m3", "bf16"])
def test_scaled_kloop_row_and_column_factors(dt):
    """The scale idioms of the reference's epilogues (06-fused-attention.py:66,78,237): a scalar and per-row
    factors, plus per-column factors, all before the cast."""
    m = compiler.analyse(jk.scaled_kloop, *scaled_sig(dt))
    assert (m.ab_dtype, m.out_dtype) == (dt, "bf16")
    assert (m.row_scale_arg, m.col_scale_arg, m.alpha) == ("rs_ptr", "cs_ptr", "alpha")
    assert (m.k_bound, m.m_bound, m.n_bound) == ("K", "M", "N")
    b = ttir.bind(m, dict(M=300, N=200, K=500, stride_am=512, stride_bk=256, stride_cm=256), (3, 2), {"alpha": 2.0})
    assert (b.m, b.n, b.k, b.lda, b.ldb, b.ldc, b.alpha, b.k_main) == (300, 200, 500, 512, 256, 256, 2.0, 384)
    assert ttir.DotKernelMatch.from_json(m.to_json()) == m


def test_scale_vector_of_other_rows_is_refused():
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16", "rs_ptr": "*fp32", "K": "i32", "stride_am": "i32",
           "stride_bk": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    with pytest.raises(ttir.NotCanonical, match="not indexed by the tile's own rows"):
        compiler.analyse(jk.wrong_scale_kloop, sig, {"BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_K": 32})
    sig["rs_ptr"] = "*fp16"
    with pytest.raises(ttir.NotCanonical):  # factors that are not fp32 in memory
        compiler.analyse(jk.wrong_scale_kloop, sig, {"BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_K": 32})


@pytest.mark.parametrize("kernel,why", [
    (jk.relu_kloop, "depends on the result of"),
    (jk.strided_k_kloop, "K elements per iteration"),
    (jk.nonzero_fill_kloop, "must be zero"),
])
def test_near_misses_are_refused(kernel, why):
    with pytest.raises(ttir.NotCanonical, match=why):
        compiler.analyse(kernel, *small_sig())


def test_casts_around_the_dot():
    """Widening the operands before the dot keeps the GEMM; narrowing them or accumulating in fp16 does not."""
    sig, cx = small_sig("bf16")
    sig32 = dict(sig, c_ptr="*fp32")
    m = compiler.analyse(jk.widened_operand_kloop, sig32, cx)
    assert (m.ab_dtype, m.out_dtype) == ("bf16", "f32")
    with pytest.raises(ttir.NotCanonical, match="narrowed from bf16 to f8E4M3FN"):
        compiler.analyse(jk.narrowed_operand_kloop, sig, cx)
    sig16, _ = small_sig("f16")
    with pytest.raises(ttir.NotCanonical, match="accumulates in f16"):
        compiler.analyse(jk.half_accumulator_kloop, sig16, cx)
    with pytest.raises(ttir.NotCanonical, match="no tensor-core path"):
        compiler.analyse(jk.plain_kloop, {"a_ptr": "*fp32", "b_ptr": "*fp32", "c_ptr": "*fp32", "K": "i32",
                                          "stride_am": "i32", "stride_ak": "constexpr", "stride_bk": "i32",
                                          "stride_bn": "constexpr", "stride_cm": "i32", "BLOCK_M": "constexpr",
                                          "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"},
                         {"stride_ak": 1, "stride_bn": 1, "BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_K": 32})


def test_side_effects_outside_the_gemm_are_refused():
    sig, cx = small_sig("bf16")
    sig = dict(list(sig.items())[:3] + [("count_ptr", "*i32")] + list(sig.items())[3:])
    with pytest.raises(ttir.NotCanonical, match="may have a side effect: tt.atomic_rmw"):
        compiler.analyse(jk.counting_kloop, sig, cx)


def test_kernels_that_are_not_gemms_are_refused_cleanly():
    with pytest.raises(ttir.NotCanonical, match="depends on the result of arith.addf"):
        compiler.analyse(jk.vector_add, {"x_ptr": "*fp32", "y_ptr": "*fp32", "out_ptr": "*fp32", "n": "i32",
                                         "BLOCK": "constexpr"}, {"BLOCK": 1024})
    with pytest.raises(ttir.NotCanonical, match="region"):
        compiler.analyse(jk.row_softmax, {"x_ptr": "*fp32", "out_ptr": "*fp32", "n_cols": "i32", "stride": "i32",
                                          "BLOCK": "constexpr"}, {"BLOCK": 1024})
    with pytest.raises(ttir.NotCanonical):
        compiler.analyse(jk.two_dots_kloop, *small_sig())
    with pytest.raises(ttir.NotCanonical, match="could not be analysed|unreadable|unknown value"):
        ttir.match_dot_kernel("module {\n  tt.func public @f(%a: i32) {\n    %x = scf.for broken {\n    }\n    tt.return\n  }\n}\n")


def test_batched_gemm_binds_one_product_per_offset_triple():
    """A base offset per program_id(2): terms of an address that are not whole blocks of the tile's own stride are
    offsets of the whole matrix; bind() groups the programs by their (A, B, C) offsets and every group must tile
    its C exactly once."""
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16", "K": "i32", "stride_ab": "i32", "stride_am": "i32",
           "stride_bb": "i32", "stride_bk": "i32", "stride_cb": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr",
           "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    m = compiler.analyse(jk.batched_kloop, sig, {"BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_K": 32})
    assert m.batch_offsets == ["pid_z*stride_ab", "pid_z*stride_bb", "pid_z*stride_cb"]
    assert (m.row0, m.col0) == ("64*pid_x", "64*pid_y")
    s = dict(K=64, stride_ab=128 * 64, stride_am=64, stride_bb=64 * 128, stride_bk=128, stride_cb=128 * 128, stride_cm=128)
    b = ttir.bind(m, s, (2, 2, 3))
    assert (b.m, b.n, b.k) == (128, 128, 64)
    assert b.batches == [(0, 0, 0), (8192, 8192, 16384), (16384, 16384, 32768)]
    with pytest.raises(ttir.NotCanonical, match="store to the same C"):
        ttir.bind(m, dict(s, stride_cb=0), (2, 2, 3))
    assert ttir.DotKernelMatch.from_json(m.to_json()) == m


def test_operand_read_at_an_offset():
    """Rows of A shifted by one against C: the product of the matrix that starts one row further down."""
    m = compiler.analyse(jk.shifted_rows_kloop, *small_sig())
    assert m.batch_offsets == ["stride_am", "0", "0"]
    b = ttir.bind(m, dict(K=64, stride_am=64, stride_bk=128, stride_cm=128), (2, 2))
    assert b.batches == [(64, 0, 0)] and (b.m, b.n, b.k) == (128, 128, 64)


def test_hand_written_ir_is_refused_with_a_reason():
    base = ttir.strip_locations(compiler.lower_to_ttir(jk.split_kloop, *split_sig()))
    with pytest.raises(ttir.NotCanonical, match="stores"):
        ttir.match_dot_kernel("\n".join(l for l in base.splitlines() if "tt.store" not in l))
    with pytest.raises(ttir.NotCanonical, match="no tt.func"):
        ttir.match_dot_kernel("module {\n}\n")


def test_triton_compile_through_the_backend():
    """triton.compile() with the b200dot target: stages source -> ttir -> b200dot, binary = the proof."""
    from triton.backends.compiler import GPUTarget
    from triton.compiler import ASTSource

    tbk.install()
    sig, cx = split_sig()
    k = triton.compile(ASTSource(jk.split_kloop, sig, cx), target=GPUTarget("b200dot", 100, 32))
    assert k.name == "split_kloop" and k.metadata.shared == 0
    assert set(k.asm) >= {"ttir", "b200dot"}
    m = ttir.DotKernelMatch.from_json(k.asm["b200dot"].decode())
    assert m == compiler.analyse(jk.split_kloop, sig, cx)
    with pytest.raises(ttir.NotCanonical):
        triton.compile(ASTSource(jk.relu_kloop, *small_sig()), target=GPUTarget("b200dot", 100, 32))


def test_backend_package_has_the_shape_triton_discovers():
    """One concrete BaseBackend in compiler.py, one concrete DriverBase in driver.py; the driver never claims
    to be the process's active driver."""
    import triton.backends as tb

    assert tb._find_concrete_subclasses(compiler, tb.BaseBackend) is compiler.B200DotBackend
    assert tb._find_concrete_subclasses(driver, tb.DriverBase) is driver.B200DotDriver
    assert driver.B200DotDriver.is_active() is False


class DryLauncher(driver.B200DotLauncher):
    calls = []

    def __call__(self, gx, gy, gz, stream, function, packed, launch_md, enter, exit_, *args):
        entry = self.prepare(function, dict(zip(self.arg_names, args)), (gx, gy, gz))
        DryLauncher.calls.append(entry)


class DryDriver(driver.B200DotDriver):
    """The real driver with the device queries answered by constants and the launcher stopped before CUDA."""

    def __init__(self):
        triton.backends.driver.DriverBase.__init__(self)
        self.utils = driver.B200DotUtils()
        self.utils.get_device_properties = lambda device: {"max_shared_mem": 232448}
        self.launcher_cls = DryLauncher
        self.get_current_device = lambda: 0
        self.set_current_device = lambda d: None
        self.get_device_capability = lambda d=0: (10, 0)
        self.get_current_stream = lambda d: 0


def test_jit_launch_reaches_the_pass_pipeline():
    """`kernel[grid](...)` end to end on CPU tensors: specialisation, compile, bind, loop_split's split point and
    dot_tile_select's tiles in the lowered loop IR."""
    from triton.runtime.driver import driver as config

    tbk.install()
    previous = config._active
    config.set_active(DryDriver())
    try:
        M, N, K = 512, 384, 4160
        a = torch.zeros(M, K, dtype=torch.bfloat16)
        b = torch.zeros(K, N, dtype=torch.bfloat16)
        c = torch.zeros(M, N, dtype=torch.bfloat16)
        DryLauncher.calls.clear()
        jk.split_kloop[(M // 128, N // 128)](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                                             c.stride(0), c.stride(1), (K // 128) * 128,
                                             BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    finally:
        config._active = previous
        jk.split_kloop.device_caches.clear()
    (entry,) = DryLauncher.calls
    bound, cfg, info = entry["bound"], entry["config"], entry["info"]
    assert (bound.m, bound.n, bound.k, bound.k_main) == (M, N, K, 4096)
    assert cfg.k_split_point == 4096
    assert info["k_main_iters"] * info["block_k"] == 4096 and info["k_tail_iters"] == 1
    assert "4096" in entry["ir"]


def test_text_helpers():
    """The pieces of the IR reader, on lines as Triton prints them."""
    line = '    %a = tt.load %p, %m, %cst : tensor<128x64x!tt.ptr<bf16>> loc(#loc12)'
    assert ttir.strip_locations(line + '\n#loc12 = loc("f.py":3:4)') == line[:-len(" loc(#loc12)")]
    nested = '%0 = arith.addi %x, %y : i32 loc(callsite(#loc3 at #loc4))'
    assert ttir.strip_locations(nested) == "%0 = arith.addi %x, %y : i32"
    assert ttir.parse_type("tensor<128x64x!tt.ptr<bf16>>") == ((128, 64), "!tt.ptr<bf16>")
    assert ttir.parse_type("tensor<1x32xi1>") == ((1, 32), "i1")
    assert ttir.parse_type("i32") == ((), "i32")
    assert ttir._split_types("{end = 128 : i32, start = 0 : i32} : tensor<128xi32>") == \
        ("{end = 128 : i32, start = 0 : i32}", "tensor<128xi32>")
    assert ttir._result_type("tensor<128xi32> -> tensor<128x1xi32>") == "tensor<128x1xi32>"
    assert ttir._result_type("tensor<64x64xf32> to tensor<64x64xbf16>") == "tensor<64x64xbf16>"
    assert ttir._result_type("tensor<8x!tt.ptr<f16>>, tensor<8xi32>") == "tensor<8x!tt.ptr<f16>>"
    assert ttir._expand_results("%2:2, %x") == ["%2#0", "%2#1", "%x"]


# ---- the reference's own lit test, when the reference tree is present --------------------------------------------

def _reference_root() -> str:
    """The reference checkout: $TRITON_EXT_REFERENCE, else a directory `reference` beside this repository."""
    import os

    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.environ.get("TRITON_EXT_REFERENCE", os.path.join(os.path.dirname(here), "reference"))


REFERENCE_LIT = _reference_root() + "/pass/LoopSplit/test/loop-split.mlir"


def _filecheck(output: str, source: str) -> list:
    """A small FileCheck: CHECK-LABEL / CHECK / CHECK-NOT in order, {{regex}}, [[VAR:regex]] and [[VAR]].
    Returns the directives that failed, in order."""
    import re

    directives = re.findall(r"//\s*(CHECK(?:-LABEL|-NOT)?):\s*(.*)", source)
    variables, pos, failed, pending_not = {}, 0, [], []

    def to_regex(pat: str) -> str:
        out, i = "", 0
        while i < len(pat):
            if pat.startswith("{{", i):
                j = pat.index("}}", i)
                out += f"(?:{pat[i + 2:j]})"
                i = j + 2
            elif pat.startswith("[[", i):
                j = pat.index("]]", i)
                body = pat[i + 2:j]
                if ":" in body:
                    name, rx = body.split(":", 1)
                    out += f"(?P<{name}>{rx.replace('.*', '[^ ,]*')})"
                else:
                    out += re.escape(variables.get(body, "<undefined>"))
                i = j + 2
            else:
                out += re.escape(pat[i])
                i += 1
        return re.sub(r"(\\ )+", r"\\s+", out)

    for kind, pat in directives:
        pat = pat.strip()
        if kind == "CHECK-NOT":
            pending_not.append(pat)
            continue
        m = re.compile(to_regex(pat)).search(output, pos)
        if not m:
            failed.append(f"{kind}: {pat}")
            continue
        for nt in pending_not:
            if re.compile(to_regex(nt)).search(output, pos, m.start()):
                failed.append(f"CHECK-NOT: {nt}")
        pending_not = []
        variables.update({k: v for k, v in m.groupdict().items() if v is not None})
        pos = m.end()
    for nt in pending_not:
        if re.compile(to_regex(nt)).search(output, pos):
            failed.append(f"CHECK-NOT: {nt}")
    return failed


def _canonicalised(text: str) -> str:
    import os
    import tempfile

    from triton._C.libtriton import ir, passes

    context = ir.context()
    ir.load_dialects(context)
    fd, path = tempfile.mkstemp(suffix=".mlir")
    try:
        with os.fdopen(fd, "w") as f:
            f.write(text)
        mod = ir.parse_mlir_module(path, context)
    finally:
        os.unlink(path)
    mod.context = context
    pm = ir.pass_manager(context)
    passes.common.add_canonicalizer(pm)
    pm.run(mod, "canonicalize")
    return ttir.strip_locations(str(mod))


@pytest.mark.skipif(not __import__("os").path.exists(REFERENCE_LIT), reason="the reference tree is not on this machine")
def test_reference_lit_test_against_the_ir_rewrite():
    """`triton-opt -triton-loop-split -canonicalize | FileCheck` of the reference's lit file
    (pass/LoopSplit/test/loop-split.mlir:1) with this package's pieces: split_loops in its as-written mode,
    Triton's canonicaliser, a small FileCheck. The four step-1 cases pass every directive. The step-10 case passes
    the loop structure but not the mid-point lines: the lit file expects `mid + (mid % step != 0)` there, the
    reference's source computes `mid + (step - mid % step)` (LoopSplit.cpp:163-167), and neither is the rounded-up
    mid point that the "intent" mode computes."""
    from triton_ext_b200.triton_backend import loop_split_ir

    cases = open(REFERENCE_LIT).read().split("// -----")
    assert len(cases) == 5
    seen = {}
    for case in cases:
        code = "\n".join(l for l in case.splitlines() if not l.strip().startswith("//"))
        label = __import__("re").search(r"@(\w+)\(", code).group(1)
        new, n = loop_split_ir.split_loops("module {\n" + code + "\n}\n", mode="as-written")
        assert n == 1, label
        out = _canonicalised(new)
        assert out.count("scf.for") == 2 and "scf.if" not in out, label
        seen[label] = _filecheck(out, case)
        # the corrected arithmetic gives verified IR of the same shape
        fixed = _canonicalised(loop_split_ir.split_loops("module {\n" + code + "\n}\n")[0])
        assert fixed.count("scf.for") == 2 and "scf.if" not in fixed, label
    step10 = seen.pop("split_kernel_step10")
    assert all(v == [] for v in seen.values()), seen
    assert len(seen) == 4
    assert step10 and step10[0].startswith("CHECK: %[[CMP:.*]] = arith.cmpi ne"), step10
    assert all("MIDP" in d or "CMP" in d or "EXT" in d for d in step10), step10  # only mid-point lines differ


REFERENCE_ATTENTION = _reference_root() + "/pass/LoopSplit/06-fused-attention.py"


def _load_reference_attention():
    """The reference's demo kernel file, executed from its text with the three queries it makes of a GPU at import
    (:28-41, :268) answered by constants. Nothing of it is written anywhere."""
    import linecache
    import re
    import types

    src = open(REFERENCE_ATTENTION).read()
    src = src.replace("DEVICE = triton.runtime.driver.active.get_active_torch_device()", 'DEVICE = "cpu"')
    src = re.sub(r"def is_hip\(\):\n    return .*\n", "def is_hip():\n    return False\n", src)
    src = re.sub(r"def is_cuda\(\):\n    return .*\n", "def is_cuda():\n    return False\n", src)
    src = src.replace("torch.cuda.get_device_capability()", "(0, 0)")
    mod = types.ModuleType("reference_fused_attention")
    mod.__file__ = REFERENCE_ATTENTION
    linecache.cache[REFERENCE_ATTENTION] = (len(src), None, src.splitlines(True), REFERENCE_ATTENTION)
    exec(compile(src, REFERENCE_ATTENTION, "exec"), mod.__dict__)
    return mod


@pytest.mark.skipif(not __import__("os").path.exists(REFERENCE_ATTENTION), reason="the reference tree is not on this machine")
@pytest.mark.parametrize("head_dim,block_m,block_n", [(64, 128, 64), (128, 128, 64)])
def test_loop_split_on_the_reference_attention_kernel(head_dim, block_m, block_n):
    """The loop LoopSplit was written for: `_attn_fwd`'s KV loop with `if start_n >= causal_start`
    (06-fused-attention.py:59-89). Its TTIR, from Triton's front end, has one scf.for, one scf.if on a compare of
    the induction variable and two tt.dot; the IR rewrite plus Triton's canonicaliser leave an off-band loop with
    neither compare nor mask and an on-band loop with the causal mask, each with both dots."""
    from triton_ext_b200.triton_backend import loop_split_ir

    fn = _load_reference_attention()._attn_fwd.fn  # below the autotuner
    sig = {"Q": "*fp16", "K": "*fp16", "V": "*fp16", "sm_scale": "fp32", "M": "*fp32", "Out": "*fp16"}
    for s in ("qz", "qh", "qm", "qk", "kz", "kh", "kn", "kk", "vz", "vh", "vk", "vn", "oz", "oh", "om", "on"):
        sig["stride_" + s] = "i32"
    sig.update({"Z": "i32", "H": "i32", "N_CTX": "i32", "HEAD_DIM": "constexpr", "BLOCK_M": "constexpr",
                "BLOCK_N": "constexpr", "CAUSAL": "constexpr"})
    cx = {"HEAD_DIM": head_dim, "BLOCK_M": block_m, "BLOCK_N": block_n, "CAUSAL": True}
    before = ttir.strip_locations(compiler.lower_to_ttir(fn, sig, cx))
    assert (before.count("scf.for"), before.count("scf.if"), before.count("tt.dot")) == (1, 1, 2)
    new, n = loop_split_ir.split_loops(before)
    assert n == 1
    after = _canonicalised(new)
    assert (after.count("scf.for"), after.count("scf.if"), after.count("tt.dot")) == (2, 0, 4)
    off_band, on_band = after.split("scf.for")[1:]
    assert "arith.cmpi" not in off_band and "arith.select" not in off_band
    assert on_band.count("arith.cmpi sge") == 1 and "arith.select" in on_band.split("tt.return")[0]
    # the K-loop matcher rightly refuses it: this is attention, not a GEMM
    with pytest.raises(ttir.NotCanonical):
        ttir.match_dot_kernel(after)


class OtherDryDriver(DryDriver):
    pass


def test_narrow_source_blocks_past_the_last_library_block():
    """K = 160 in source blocks of 32 (all whole) but library blocks of 64: the split handed to the passes is 128."""
    launcher = driver.B200DotLauncher.__new__(driver.B200DotLauncher)
    launcher.arg_names, launcher._bound, launcher.launches = [], {}, 0
    sig = {"a_ptr": "*bf16", "b_ptr": "*bf16", "c_ptr": "*bf16", "K": "i32", "stride_ab": "i32", "stride_am": "i32",
           "stride_bb": "i32", "stride_bk": "i32", "stride_cb": "i32", "stride_cm": "i32", "BLOCK_M": "constexpr",
           "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    m = compiler.analyse(jk.batched_kloop, sig, {"BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_K": 32})
    values = dict(K=160, stride_ab=256 * 160, stride_am=160, stride_bb=160 * 192, stride_bk=192, stride_cb=256 * 192,
                  stride_cm=192)
    entry = launcher.prepare(m, values, (4, 3, 2))
    assert entry["bound"].k_main == 160 and entry["config"].k_split_point == 128
    assert len(entry["bound"].batches) == 2


def test_host_tensor_descriptors_through_a_jit_launch():
    """Descriptors built on the host and passed as arguments (the form of the reference's `_attn_fwd_tma`,
    06-fused-attention.py:275-329): shapes and strides are read from the descriptor objects at launch, and the three
    descriptors must agree on M, N and K."""
    from triton.runtime.driver import driver as config
    from triton.tools.tensor_descriptor import TensorDescriptor

    sig = {"a_desc": "tensordesc<bf16[128,64]>", "b_desc": "tensordesc<bf16[64,128]>", "c_desc": "tensordesc<bf16[128,128]>",
           "K": "i32", "BLOCK_M": "constexpr", "BLOCK_N": "constexpr", "BLOCK_K": "constexpr"}
    m = compiler.analyse(jk.host_descriptor_kloop, sig, {"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 64})
    assert (m.a_arg, m.k_bound, m.m_bound, m.n_bound) == ("a_desc", "a_desc__shape1", "c_desc__shape0", "c_desc__shape1")
    assert [e[0] for e in m.equal_at_launch] == ["K", "M", "N"]

    M, N, K = 300, 200, 504
    a = torch.zeros(M, K, dtype=torch.bfloat16)
    b = torch.zeros(K, N, dtype=torch.bfloat16)
    c = torch.zeros(M, N, dtype=torch.bfloat16)
    desc = lambda t, blk: TensorDescriptor(t, list(t.shape), list(t.stride()), blk)
    kernel = triton.jit(jk.host_descriptor_kloop.fn)
    tbk.install()
    previous = config._active
    config.set_active(DryDriver())
    try:
        DryLauncher.calls.clear()
        kernel[(3, 2)](desc(a, [128, 64]), desc(b, [64, 128]), desc(c, [128, 128]), K, BLOCK_M=128, BLOCK_N=128, BLOCK_K=64)
        (entry,) = DryLauncher.calls
        assert (entry["bound"].m, entry["bound"].n, entry["bound"].k, entry["bound"].lda) == (M, N, K, K)
        with pytest.raises(ttir.NotCanonical, match="disagree on K"):
            kernel[(3, 2)](desc(a, [128, 64]), desc(torch.zeros(K + 8, N, dtype=torch.bfloat16), [64, 128]),
                           desc(c, [128, 128]), K, BLOCK_M=128, BLOCK_N=128, BLOCK_K=64)
    finally:
        config._active = previous


def test_jit_keeps_one_cache_per_driver():
    """triton_backend.jit: the same kernel object under two drivers in turn, each with its own compile cache."""
    from triton.runtime.driver import driver as config

    tbk.install()
    kernel = tbk.jit(jk.split_kloop.fn)
    a = torch.zeros(128, 256, dtype=torch.bfloat16)
    b = torch.zeros(256, 128, dtype=torch.bfloat16)
    c = torch.zeros(128, 128, dtype=torch.bfloat16)
    previous = config._active
    try:
        for drv in (DryDriver(), OtherDryDriver(), DryDriver()):
            config.set_active(drv)
            DryLauncher.calls.clear()
            kernel[(1, 1)](a, b, c, 128, 128, 256, 256, 1, 128, 1, 128, 1, 256, BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
            assert len(DryLauncher.calls) == 1 and DryLauncher.calls[0]["bound"].k == 256
    finally:
        config._active = previous
    assert set(kernel._caches_by_driver) == {"DryDriver", "OtherDryDriver"}
    assert all(len(v[0][0]) == 1 for v in kernel._caches_by_driver.values())  # one compiled kernel per driver, device 0


def test_tile_origins_agree_with_the_kernels_own_arithmetic():
    """The symbolic tile origin, evaluated numerically over a whole grid, against a direct Python transcription of
    grouped_masked_kloop's program-id arithmetic, over random shapes (hypothesis)."""
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    m = compiler.analyse(jk.grouped_masked_kloop, *grouped_sig())

    @settings(max_examples=60, deadline=None)
    @given(M=st.integers(1, 3000), N=st.integers(1, 3000), extra=st.integers(0, 3))
    def check(M, N, extra):
        tiles_m, tiles_n = -(-M // 64), -(-N // 128)
        grid = tiles_m * tiles_n
        rows, cols, _ = ttir._tile_origins(m, dict(M=M, N=N, K=64, stride_am=64, stride_bn=64, stride_cm=N), (grid, 1, 1))
        for pid in {0, grid - 1, grid // 2, min(grid - 1, extra)}:
            per_group = 4 * tiles_n
            first_m = (pid // per_group) * 4
            rows_here = min(tiles_m - first_m, 4)
            pid_m = first_m + (pid % per_group) % rows_here
            pid_n = (pid % per_group) // rows_here
            assert (rows[pid], cols[pid]) == (pid_m * 64, pid_n * 128), (M, N, pid)
        b = ttir.bind(m, dict(M=M, N=N, K=64, stride_am=64, stride_bn=64, stride_cm=N), (grid,), {"alpha": 1.0})
        assert (b.m, b.n) == (M, N)

    check()


def test_loop_split_text_preserves_meaning_on_random_loops():
    """Random lower bound, upper bound, step, comparand, predicate and operand order (hypothesis): the bisected IR
    computes what the original computes (intent mode; the as-written mode is known not to, for sgt / sle and for
    distances that are already multiples of the step)."""
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    from triton_ext_b200.triton_backend import loop_split_ir

    @settings(max_examples=150, deadline=None)
    @given(lo=st.integers(-6, 12), n=st.integers(-4, 40), c=st.integers(-10, 45), step=st.integers(1, 9),
           pred=st.sampled_from(["slt", "sle", "sgt", "sge"]), swap=st.booleans())
    def check(lo, n, c, step, pred, swap):
        text = (LIT_CASE.replace("STEP", str(step)).replace("PRED", pred)
                .replace("LHS", "%c" if swap else "%i").replace("RHS", "%i" if swap else "%c")
                .replace("%c0 = arith.constant 0 : i32", f"%c0 = arith.constant {lo} : i32\n    %zero = arith.constant 0 : i32")
                .replace("iter_args(%acc = %c0)", "iter_args(%acc = %zero)"))
        new, k = loop_split_ir.split_loops(text)
        assert k == 1
        assert run_scalar_ir(new, n, c) == run_scalar_ir(text, n, c)

    check()

    # Unsigned compares: split (behind a run-time guard on the comparand's sign bit) only when the lower bound is a
    # non-negative constant; with a negative lower bound the compare is not monotone in the induction variable and the
    # loop is left alone. Either way the meaning is kept, for negative comparands too.
    @settings(max_examples=200, deadline=None)
    @given(lo=st.integers(-6, 12), n=st.integers(-4, 40), c=st.one_of(st.integers(-10, 45), st.sampled_from([-1, -2**31])),
           step=st.integers(1, 9), pred=st.sampled_from(["ult", "ule", "ugt", "uge"]), swap=st.booleans())
    def check_unsigned(lo, n, c, step, pred, swap):
        text = (LIT_CASE.replace("STEP", str(step)).replace("PRED", pred)
                .replace("LHS", "%c" if swap else "%i").replace("RHS", "%i" if swap else "%c")
                .replace("%c0 = arith.constant 0 : i32", f"%c0 = arith.constant {lo} : i32\n    %zero = arith.constant 0 : i32")
                .replace("iter_args(%acc = %c0)", "iter_args(%acc = %zero)"))
        new, k = loop_split_ir.split_loops(text)
        assert k == (1 if lo >= 0 else 0)
        assert run_scalar_ir(new, n, c) == run_scalar_ir(text, n, c)

    check_unsigned()


def test_as_written_mode_reproduces_the_reference_and_its_off_by_one():
    """The as-written rewrite follows the reference's arithmetic to the letter, including where that changes what the
    loop computes: `iv > c` is split at c (the iteration iv == c lands in the loop whose compare reads true), a
    comparand beyond the upper bound makes the first loop run past it, and a distance that is already a multiple of
    the step is pushed one step further. The intent mode is exact on both."""
    from triton_ext_b200.triton_backend import loop_split_ir

    def case(pred, step):
        return (LIT_CASE.replace("STEP", str(step)).replace("PRED", pred).replace("LHS", "%i").replace("RHS", "%c"))

    sgt = case("sgt", 1)
    written, _ = loop_split_ir.split_loops(sgt, mode="as-written")
    exact, _ = loop_split_ir.split_loops(sgt)
    assert run_scalar_ir(exact, 10, 5) == run_scalar_ir(sgt, 10, 5)
    assert run_scalar_ir(written, 10, 5) != run_scalar_ir(sgt, 10, 5)
    assert run_scalar_ir(written, 10, 20) != run_scalar_ir(sgt, 10, 20)      # no clamping: the first loop runs past hi
    assert run_scalar_ir(exact, 10, 20) == run_scalar_ir(sgt, 10, 20)
    slt = case("slt", 1)
    written, _ = loop_split_ir.split_loops(slt, mode="as-written")
    assert run_scalar_ir(written, 10, 5) == run_scalar_ir(slt, 10, 5)        # the case the pass was written for
    step10 = case("slt", 10)
    written, _ = loop_split_ir.split_loops(step10, mode="as-written")
    exact, _ = loop_split_ir.split_loops(step10)
    assert run_scalar_ir(exact, 100, 20) == run_scalar_ir(step10, 100, 20)
    assert run_scalar_ir(written, 100, 20) != run_scalar_ir(step10, 100, 20)   # mid 20 -> 30: iteration 20 reads true
    assert run_scalar_ir(written, 100, 25) == run_scalar_ir(step10, 100, 25)   # mid 25 -> 30: correct
