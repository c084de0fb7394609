"""The arithmetic-intensity analysis (no GPU): what it picks for the BASELINE configurations, that
explicit settings are respected, and the C-ABI's argument checking."""
import ctypes

import pytest
import torch

from triton_ext_b200 import backend as B

bf16, f16, f8, f32 = torch.bfloat16, torch.float16, torch.float8_e4m3fn, torch.float32


def test_library_loads_without_a_gpu(built_libs):
    lib = B.load_library()
    assert lib.tx_dot_device_count() >= 0
    assert B.kernel_launches() >= 0


def test_compute_bound_shapes_get_cta_pairs_and_big_tiles(built_libs):
    """Tensor-bound shapes run on CTA pairs. Where 256 x 512 tiles cover the problem without padding and in no more
    machine time than 256 x 256 tiles (one wide wave = two narrow ones), the wide tile is chosen (measured 2.4 % faster);
    fp8 operands and
    the column panels of the sharded GEMM (which quantise worse with it) keep 256 x 256 tiles with two K atoms per stage."""
    want_wide = {(4096, 4096, 4160): True, (8192, 8192, 8192): False, (8192, 8192, 4160): True, (16384, 28672, 8192): False, (16384, 3584, 8192): False,
                 (16384, 7168, 8192): False, (2048, 2048, 2048): False}
    for (m, n, k), wide in want_wide.items():
        dt = f8 if (m, n, k) == (8192, 8192, 8192) else bf16
        info = B.preview(B.make_problem(m, n, k, dt, bf16))
        assert info["cta_pair"] == 1 and info["block_m"] == 256 and info["swap_ab"] == 0, (m, n, k, info)
        assert info["block_n"] == (512 if wide else 256), (m, n, k, info)
        assert info["smem_bytes"] <= 227 * 1024 and info["tmem_columns"] == 512
        atoms = info["block_k"] * (1 if dt == f8 else 2) // 128
        assert (atoms, info["stages"]) == ((1, 4) if wide else (2, 3)), (m, n, k, info)
    # an explicit request is honoured on any pair-sized problem; the wide tile has no stream-K or deep-block form
    assert B.preview(B.make_problem(16384, 3584, 8192, bf16, bf16), B.make_config(block_n=512))["block_n"] == 512
    for kw in (dict(block_n=512, schedule=B.TXD_SCHED_STREAM_K), dict(block_n=512, atoms=2), dict(block_n=512, cta_pair=2)):
        with pytest.raises(B.DotError):
            B.preview(B.make_problem(4096, 4096, 4096, bf16, bf16), B.make_config(**kw))


def test_decode_shape_is_swapped(built_libs):
    """m = 16: the 14336-wide side feeds the 128 TMEM lanes (swap), block_n = 16, deep K blocks so that few
    TMA copies are issued per byte; whole tiles (measured faster than stream-K here: the fix-up costs more
    than the 36 idle SMs)."""
    info = B.preview(B.make_problem(16, 14336, 4096, bf16, bf16))
    assert info["swap_ab"] == 1 and info["block_n"] == 16 and info["cta_pair"] == 0
    assert info["block_k"] >= 128 and info["grid"] == 112
    assert info["algorithmic_bytes"] == 16 * 4096 * 2 + 4096 * 14336 * 2 + 16 * 14336 * 2
    forced = B.preview(B.make_problem(16, 14336, 4096, bf16, bf16), B.make_config(schedule=B.TXD_SCHED_STREAM_K))
    assert forced["grid"] == 148 and forced["scratch_bytes"] > 0


def test_measured_rules_of_the_tile_model(built_libs):
    """Three choices that come from measurements, not from the model's arithmetic: an operand ring of at most 200 KiB,
    raster groups twice as tall where their P panels then still fit 32 MiB of L2, and an evenly dividing grid for
    HBM-bound whole-tile schedules."""
    cfg3 = B.preview(B.make_problem(16, 14336, 4096, bf16, bf16))
    assert cfg3["stages"] == 5 and cfg3["stages"] * 36 * 1024 <= 200 * 1024 < 6 * 36 * 1024
    assert B.preview(B.make_problem(16, 14336, 4096, bf16, bf16), B.make_config(stages=6))["stages"] == 6   # a request is honoured
    cfg4 = B.preview(B.make_problem(8192, 8192, 8192, f8, bf16))
    assert cfg4["group_m"] == 16          # 16 x 256 rows x 8192 bytes = 32 MiB
    cfg5 = B.preview(B.make_problem(16384, 28672, 8192, bf16, bf16))
    assert cfg5["group_m"] == 8 and cfg5["grid"] == 148      # 8 rows already hold 32 MiB; tensor-bound keeps every SM
    skinny = B.preview(B.make_problem(16, 28672, 8192, bf16, bf16))
    assert skinny["schedule"] == B.TXD_SCHED_DATA_PARALLEL and skinny["grid"] == 112      # 224 tiles = 2 x 112
    assert B.preview(B.make_problem(16, 28672, 8192, bf16, bf16), B.make_config(group_m=4))["group_m"] == 4


def test_split_point_fields(built_libs):
    info = B.preview(B.make_problem(4096, 4096, 4160, bf16, bf16), B.make_config(atoms=1))
    assert (info["k_main_iters"], info["k_tail_iters"], info["k_tail_mmas"]) == (65, 0, 4)
    info = B.preview(B.make_problem(4096, 4096, 4160, bf16, bf16), B.make_config(atoms=1, k_split_point=4096))
    assert (info["k_main_iters"], info["k_tail_iters"], info["k_tail_mmas"]) == (64, 1, 4)
    # two atoms per stage: the physical K block is BLOCK_K = 128, main 32 blocks + a 64-wide remainder
    info = B.preview(B.make_problem(4096, 4096, 4160, bf16, bf16), B.make_config(atoms=2))
    assert (info["block_k"], info["k_main_iters"], info["k_tail_iters"], info["k_tail_mmas"]) == (128, 32, 1, 4)
    info = B.preview(B.make_problem(256, 256, 200, bf16, bf16))
    assert (info["k_main_iters"], info["k_tail_iters"], info["k_tail_mmas"]) == (3, 1, 1)  # 200 = 3*64 + 8
    info = B.preview(B.make_problem(256, 256, 200, bf16, bf16), B.make_config(k_split_point=-1))
    assert (info["k_main_iters"], info["k_tail_iters"]) == (0, 4)
    with pytest.raises(B.DotError) as e:
        B.preview(B.make_problem(256, 256, 200, bf16, bf16), B.make_config(k_split_point=256))
    assert e.value.status == B.TXD_ERR_INVALID


def test_explicit_config_is_kept(built_libs):
    info = B.preview(B.make_problem(1024, 1024, 1024, bf16, bf16),
                     B.make_config(block_n=64, stages=3, cta_pair=2, schedule=2, group_m=2, max_ctas=40))
    assert (info["block_n"], info["stages"], info["cta_pair"], info["schedule"], info["group_m"]) == (64, 3, 0, 2, 2)
    assert info["grid"] <= 40
    with pytest.raises(B.DotError):
        B.preview(B.make_problem(1024, 1024, 1024, bf16, bf16), B.make_config(block_n=256, stages=12))  # ring too big


def test_argument_checks(built_libs):
    bad = [
        (B.make_problem(-1, 8, 8, bf16, bf16), B.TXD_ERR_INVALID),
        (B.make_problem(64, 64, 64, f32, f32), B.TXD_ERR_UNSUPPORTED),       # fp32 operands are not tt.dot tensor-core types
        (B.make_problem(64, 64, 64, bf16, f8), B.TXD_ERR_UNSUPPORTED),       # fp8 output
        (B.make_problem(64, 64, 60, bf16, bf16), B.TXD_ERR_UNSUPPORTED),     # lda = 60: rows not 16-byte aligned
        (B.make_problem(64, 60, 64, bf16, bf16), B.TXD_ERR_UNSUPPORTED),     # ldb = 60
        (B.make_problem(64, 64, 64, bf16, bf16, lda=32), B.TXD_ERR_INVALID),  # lda < k
    ]
    for pr, status in bad:
        with pytest.raises(B.DotError) as e:
            B.preview(pr)
        assert e.value.status == status, B.load_library().tx_dot_last_error()
    info = B.PlanInfo()
    assert B.load_library().tx_dot_plan_preview(None, None, 148, ctypes.byref(info)) == B.TXD_ERR_INVALID
    # empty problems are legal and need no kernel
    assert B.preview(B.make_problem(0, 64, 64, bf16, bf16))["grid"] == 0


def test_no_gpu_means_no_compute(built_libs):
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(B.DotError) as e:
        B.DotPlan(B.make_problem(128, 128, 128, bf16, bf16))
    assert e.value.status == B.TXD_ERR_NO_DEVICE
    with pytest.raises(ValueError):
        B.dot(torch.zeros(8, 8, dtype=bf16), torch.zeros(8, 8, dtype=bf16))
