"""@triton.jit K-loop kernels launched through the b200dot Triton backend on a B200, against torch fp32
matmul, against the library's own entry point (bit-exact: same kernel), and against the same kernel object
compiled by Triton's stock CUDA backend (the reference's lowering of tt.dot)."""
import math

import pytest
import torch

triton = pytest.importorskip("triton")

import jit_kernels as jk  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _fresh_kernels():
    yield
    for fn in (jk.split_kloop, jk.grouped_masked_kloop, jk.plain_kloop, jk.scaled_kloop, jk.wrapped_kloop, jk.persistent_kloop, jk.descriptor_kloop, jk.nt_kloop):
        fn.device_caches.clear()


def _rand(shape, dtype, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype).to(device)


def _launch_split(a, b, c, k_main, bm=128, bn=128, bk=128):
    M, K = a.shape
    N = b.shape[1]
    jk.split_kloop[(math.ceil(M / bm), math.ceil(N / bn))](
        a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1), k_main,
        BLOCK_M=bm, BLOCK_N=bn, BLOCK_K=bk)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1024, 512, 4160), (256, 384, 200)])
def test_split_kloop_through_backend(built_libs, cuda_device, dtype, shape):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = shape
    a, b = _rand((M, K), dtype, cuda_device, 1), _rand((K, N), dtype, cuda_device, 2)
    c = torch.full((M, N), float("nan"), dtype=dtype, device=cuda_device)
    before = backend.kernel_launches()
    with tbk.activate():
        _launch_split(a, b, c, (K // 128) * 128)
        _launch_split(a, b, c, (K // 128) * 128)  # second launch: cached compile and plan
    torch.cuda.synchronize()
    assert backend.kernel_launches() - before == 2
    ref = a.float() @ b.float()
    torch.testing.assert_close(c.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    assert torch.equal(c, backend.dot(a, b, check=True))


def test_transposed_views_and_early_split(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 384, 256, 1000
    a = _rand((K, M), torch.float16, cuda_device, 3).t()   # column-major A
    b = _rand((N, K), torch.float16, cuda_device, 4).t()   # column-major B
    c = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
    with tbk.activate():
        _launch_split(a, b, c, 512)   # split point well before the last full block
    torch.cuda.synchronize()
    assert torch.equal(c, backend.dot(a, b, check=True))
    with tbk.activate(), pytest.raises(tbk.NotCanonical, match="unmasked load run past"):
        _launch_split(a, b, c, 1024)


def test_grouped_masked_kloop_ragged(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 1000, 304, 1112
    a = _rand((M, K), torch.float16, cuda_device, 5)
    b = _rand((N, K), torch.float16, cuda_device, 6).t()
    c = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
    grid = (math.ceil(M / 64) * math.ceil(N / 128),)
    with tbk.activate():
        jk.grouped_masked_kloop[grid](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                                      c.stride(0), c.stride(1), 0.5, BLOCK_M=64, BLOCK_N=128, BLOCK_K=32, GROUP=4)
    torch.cuda.synchronize()
    ref = 0.5 * (a.float() @ b.float())
    torch.testing.assert_close(c.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    assert torch.equal(c, backend.dot(a, b, alpha=0.5, check=True))


def test_plain_kloop_fp32_out(built_libs, cuda_device):
    from triton_ext_b200 import triton_backend as tbk

    M, N, K = 384, 320, 512
    a, b = _rand((M, K), torch.bfloat16, cuda_device, 7), _rand((K, N), torch.bfloat16, cuda_device, 8)
    c = torch.empty((M, N), dtype=torch.float32, device=cuda_device)
    with tbk.activate():
        jk.plain_kloop[(N // 64, M // 128)](a, b, c, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0),
                                            BLOCK_M=128, BLOCK_N=64, BLOCK_K=64)
    torch.cuda.synchronize()
    torch.testing.assert_close(c, a.float() @ b.float(), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.bfloat16])
def test_scaled_kloop_with_row_and_column_factors(built_libs, cuda_device, dtype):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 300, 208, 528
    a, b = _rand((M, K), dtype, cuda_device, 11), _rand((K, N), dtype, cuda_device, 12)
    rs = torch.rand(M, device=cuda_device) + 0.5
    cs = torch.rand(N, device=cuda_device) + 0.5
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    with tbk.activate():
        jk.scaled_kloop[(math.ceil(M / 128), math.ceil(N / 128))](
            a, b, c, rs, cs, M, N, K, a.stride(0), b.stride(0), c.stride(0), 0.25,
            BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    torch.cuda.synchronize()
    ref = 0.25 * rs[:, None] * cs[None, :] * (a.float() @ b.float())
    tol = 3e-2 if dtype == torch.float8_e4m3fn else 1e-2
    torch.testing.assert_close(c.float(), ref, rtol=tol, atol=tol * ref.abs().max().item())
    assert torch.equal(c, backend.dot(a, b, out_dtype=torch.bfloat16, row_scale=rs, col_scale=cs, alpha=0.25, check=True))


def test_wrapped_kloop_ragged(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 300, 200, 504
    a, b = _rand((M, K), torch.float16, cuda_device, 13), _rand((K, N), torch.float16, cuda_device, 14)
    c = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
    with tbk.activate():
        jk.wrapped_kloop[(math.ceil(M / 128) * math.ceil(N / 64),)](
            a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1),
            BLOCK_M=128, BLOCK_N=64, BLOCK_K=64)
    torch.cuda.synchronize()
    assert torch.equal(c, backend.dot(a, b, check=True))
    ref = a.float() @ b.float()
    torch.testing.assert_close(c.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())


def test_persistent_kloop(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 1000, 776, 520
    a, b = _rand((M, K), torch.bfloat16, cuda_device, 17), _rand((K, N), torch.bfloat16, cuda_device, 18)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    programs = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    with tbk.activate():
        jk.persistent_kloop[(programs,)](a, b, c, M, N, K, a.stride(0), b.stride(0), c.stride(0),
                                         BLOCK_M=128, BLOCK_N=128, BLOCK_K=64, GROUP=8)
    torch.cuda.synchronize()
    assert torch.equal(c, backend.dot(a, b, check=True))
    ref = a.float() @ b.float()
    torch.testing.assert_close(c.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())


def test_descriptor_kloop(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 300, 200, 504
    a, b = _rand((M, K), torch.bfloat16, cuda_device, 19), _rand((K, N), torch.bfloat16, cuda_device, 20)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    with tbk.activate():
        jk.descriptor_kloop[(math.ceil(M / 128), math.ceil(N / 128))](
            a, b, c, M, N, K, a.stride(0), b.stride(0), c.stride(0), BLOCK_M=128, BLOCK_N=128, BLOCK_K=64)
    torch.cuda.synchronize()
    assert torch.equal(c, backend.dot(a, b, check=True))


def test_packaged_kernel_ragged(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk
    from triton_ext_b200.triton_backend import kernels

    M, N, K = 777, 333, 1096
    a, b = _rand((M, K), torch.float16, cuda_device, 21), _rand((K, N), torch.float16, cuda_device, 22)
    b = b.t().contiguous().t()  # column-major B
    c = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
    try:
        with tbk.activate():
            kernels.launch_dot_kloop(a, b, c)
        torch.cuda.synchronize()
    finally:
        kernels.dot_kloop.device_caches.clear()
    assert torch.equal(c, backend.dot(a, b, check=True))


def test_nt_kloop(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 300, 200, 504
    a, bt = _rand((M, K), torch.bfloat16, cuda_device, 23), _rand((N, K), torch.bfloat16, cuda_device, 24)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    with tbk.activate():
        jk.nt_kloop[(math.ceil(M / 128), math.ceil(N / 64))](a, bt, c, M, N, K, a.stride(0), bt.stride(0), c.stride(0),
                                                             BLOCK_M=128, BLOCK_N=64, BLOCK_K=64)
    torch.cuda.synchronize()
    assert torch.equal(c, backend.dot(a, bt.t(), check=True))


def test_autotuned_kernel(built_libs, cuda_device):
    """@triton.autotune over block shapes: every configuration compiles to a proof of the same GEMM, the tuner's
    benchmark runs through the backend's launcher, the result does not depend on the winner."""
    from triton_ext_b200 import backend, triton_backend as tbk

    tuned = triton.autotune(
        configs=[triton.Config({"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 64}, num_warps=4, num_stages=3),
                 triton.Config({"BLOCK_M": 64, "BLOCK_N": 256, "BLOCK_K": 32}, num_warps=8, num_stages=4)],
        key=["M", "N", "K"])(triton.jit(jk.grouped_masked_kloop.fn))
    M, N, K = 520, 776, 1096
    a, b = _rand((M, K), torch.float16, cuda_device, 25), _rand((K, N), torch.float16, cuda_device, 26)
    c = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
    grid = lambda meta: (math.ceil(M / meta["BLOCK_M"]) * math.ceil(N / meta["BLOCK_N"]),)
    with tbk.activate():
        tuned[grid](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1), 1.0,
                    GROUP=4)
    torch.cuda.synchronize()
    assert tuned.best_config is not None
    assert torch.equal(c, backend.dot(a, b, check=True))


def test_per_driver_jit_alternates_between_lowerings(built_libs, cuda_device):
    """triton_backend.jit: one kernel object launched under Triton's stock driver, this backend, and the stock
    driver again, without touching its caches; all three results agree."""
    from triton_ext_b200 import triton_backend as tbk

    kernel = tbk.jit(jk.split_kloop.fn)
    M, N, K = 256, 256, 576
    a, b = _rand((M, K), torch.bfloat16, cuda_device, 27), _rand((K, N), torch.bfloat16, cuda_device, 28)
    outs = [torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device) for _ in range(3)]

    def launch(c):
        kernel[(M // 64, N // 64)](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                                   c.stride(0), c.stride(1), 576, BLOCK_M=64, BLOCK_N=64, BLOCK_K=64)

    try:
        launch(outs[0])
        torch.cuda.synchronize()
    except Exception as e:  # the stock tool chain (ptxas) is not part of this package
        pytest.skip(f"Triton's CUDA backend could not compile here: {type(e).__name__}")
    with tbk.activate():
        launch(outs[1])
    launch(outs[2])
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[2])
    scale = (a.float() @ b.float()).abs().max().item()
    assert (outs[1].float() - outs[0].float()).abs().max().item() <= 2.0 ** -7 * scale
    assert set(kernel._caches_by_driver) == {"CudaDriver", "B200DotDriver"}


def test_batched_kloop(built_libs, cuda_device):
    """Four matrix products in one launch (program_id(2) picks the matrices): one library launch each."""
    from triton_ext_b200 import backend, triton_backend as tbk

    B, M, N, K = 4, 256, 192, 160
    a = _rand((B, M, K), torch.bfloat16, cuda_device, 29)
    b = _rand((B, K, N), torch.bfloat16, cuda_device, 30)
    c = torch.full((B, M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    before = backend.kernel_launches()
    kernel = triton.jit(jk.batched_kloop.fn)
    with tbk.activate():
        kernel[(M // 64, N // 64, B)](a, b, c, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0),
                                      c.stride(1), BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    torch.cuda.synchronize()
    assert backend.kernel_launches() - before == B
    for i in range(B):
        assert torch.equal(c[i], backend.dot(a[i], b[i], check=True)), i
    ref = torch.bmm(a.float(), b.float())
    torch.testing.assert_close(c.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())


def test_operand_at_an_offset(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 128, 128, 64
    a = _rand((M + 8, K), torch.bfloat16, cuda_device, 31)   # the kernel reads rows 1 .. M of it
    b = _rand((K, N), torch.bfloat16, cuda_device, 32)
    c = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
    kernel = triton.jit(jk.shifted_rows_kloop.fn)
    with tbk.activate():
        kernel[(M // 64, N // 64)](a, b, c, K, a.stride(0), b.stride(0), c.stride(0), BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    torch.cuda.synchronize()
    ref = a[1:M + 1].float() @ b.float()
    torch.testing.assert_close(c.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())


def test_block_pointer_kloop(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 300, 200, 504
    a, b = _rand((M, K), torch.bfloat16, cuda_device, 33), _rand((K, N), torch.bfloat16, cuda_device, 34)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    kernel = triton.jit(jk.block_pointer_kloop.fn)
    with tbk.activate():
        kernel[(math.ceil(M / 128), math.ceil(N / 64))](a, b, c, M, N, K, a.stride(0), b.stride(0), c.stride(0),
                                                         BLOCK_M=128, BLOCK_N=64, BLOCK_K=64)
    torch.cuda.synchronize()
    assert torch.equal(c, backend.dot(a, b, check=True))


def test_single_dot_fp8_e5m2(built_libs, cuda_device):
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 100, 80, 96
    a, b = _rand((M, K), torch.float8_e5m2, cuda_device, 35), _rand((K, N), torch.float8_e5m2, cuda_device, 36)
    c = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
    kernel = triton.jit(jk.single_dot.fn)
    with tbk.activate():
        kernel[(2, 2)](a, b, c, M, N, K, a.stride(0), b.stride(0), c.stride(0), BLOCK_M=64, BLOCK_N=64, BLOCK_K=128)
    torch.cuda.synchronize()
    ref = a.float() @ b.float()
    torch.testing.assert_close(c.float(), ref, rtol=3e-2, atol=3e-2 * ref.abs().max().item())
    assert torch.equal(c, backend.dot(a, b, out_dtype=torch.float16, check=True))


def test_column_major_output(built_libs, cuda_device):
    from triton_ext_b200 import triton_backend as tbk

    M, N, K = 256, 384, 200
    a, b = _rand((M, K), torch.float16, cuda_device, 37), _rand((K, N), torch.float16, cuda_device, 38)
    c = torch.full((N, M), float("nan"), dtype=torch.float16, device=cuda_device).t()   # [M, N] view, column-major
    kernel = triton.jit(jk.split_kloop.fn)
    with tbk.activate():
        kernel[(M // 128, N // 128)](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                                     c.stride(0), c.stride(1), 128, BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    torch.cuda.synchronize()
    ref = a.float() @ b.float()
    torch.testing.assert_close(c.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())


def test_host_descriptor_kloop(built_libs, cuda_device):
    from triton.tools.tensor_descriptor import TensorDescriptor
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 300, 200, 504
    a, b = _rand((M, K), torch.bfloat16, cuda_device, 39), _rand((K, N), torch.bfloat16, cuda_device, 40)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    desc = lambda t, blk: TensorDescriptor(t, list(t.shape), list(t.stride()), blk)
    kernel = triton.jit(jk.host_descriptor_kloop.fn)
    with tbk.activate():
        kernel[(3, 2)](desc(a, [128, 64]), desc(b, [64, 128]), desc(c, [128, 128]), K, BLOCK_M=128, BLOCK_N=128, BLOCK_K=64)
    torch.cuda.synchronize()
    assert torch.equal(c, backend.dot(a, b, check=True))


def test_launch_inside_a_cuda_graph(built_libs, cuda_device):
    """After one eager launch (compile, plan) the same launch is capturable: nothing allocates or synchronises."""
    from triton_ext_b200 import backend, triton_backend as tbk

    M, N, K = 512, 256, 1096
    a, b = _rand((M, K), torch.bfloat16, cuda_device, 15), _rand((K, N), torch.bfloat16, cuda_device, 16)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=cuda_device)
    with tbk.activate():
        _launch_split(a, b, c, 1024)
        torch.cuda.synchronize()
        want = c.clone()
        c.zero_()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                _launch_split(a, b, c, 1024)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
    assert torch.equal(c, want) and torch.equal(c, backend.dot(a, b, check=True))


def test_cpu_tensors_are_refused(built_libs, cuda_device):
    from triton_ext_b200 import triton_backend as tbk

    a = torch.zeros(128, 128, dtype=torch.bfloat16)
    with tbk.activate(), pytest.raises(TypeError, match="CUDA tensor"):
        _launch_split(a, a.clone(), a.clone(), 128)


def test_same_kernel_under_triton_cuda_backend(built_libs, cuda_device):
    """One kernel object, two lowerings: Triton's own code generation for tt.dot, then this backend."""
    from triton_ext_b200 import triton_backend as tbk

    M, N, K = 512, 384, 1088 + 64
    a, b = _rand((M, K), torch.bfloat16, cuda_device, 9), _rand((K, N), torch.bfloat16, cuda_device, 10)
    c_triton = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
    c_ours = torch.empty_like(c_triton)
    try:
        _launch_split(a, b, c_triton, (K // 64) * 64, bm=64, bn=64, bk=64)
        torch.cuda.synchronize()
    except Exception as e:  # the stock tool chain (ptxas) is not part of this package
        pytest.skip(f"Triton's CUDA backend could not compile here: {type(e).__name__}")
    jk.split_kloop.device_caches.clear()
    with tbk.activate():
        _launch_split(a, b, c_ours, (K // 64) * 64, bm=64, bn=64, bk=64)
    torch.cuda.synchronize()
    ref = a.float() @ b.float()
    scale = ref.abs().max().item()
    assert (c_triton.float() - ref).abs().max().item() <= 1e-2 * scale
    assert (c_ours.float() - ref).abs().max().item() <= 1e-2 * scale
    # both round an fp32 accumulation of the same products to bf16: at most one unit in the last place apart
    assert (c_ours.float() - c_triton.float()).abs().max().item() <= 2.0 ** -7 * scale
