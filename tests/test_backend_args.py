"""Argument checks of the Python binding that must fire before any launch (they need no GPU): a mistyped or
mis-sized output buffer or scale vector would otherwise be written or read past its end by the kernel."""
import pytest
import torch

from triton_ext_b200 import backend as B

bf16, f32 = torch.bfloat16, torch.float32


def ab(m=32, n=48, k=64):
    return torch.zeros(m, k, dtype=bf16), torch.zeros(k, n, dtype=bf16)


def test_out_shape_dtype_are_checked_before_anything_else():
    a, b = ab()
    with pytest.raises(ValueError, match="shape"):
        B.dot(a, b, out=torch.zeros(32, 40, dtype=bf16))
    with pytest.raises(TypeError, match="out_dtype"):
        B.dot(a, b, out=torch.zeros(32, 48, dtype=bf16), out_dtype=f32)      # fp32 results into a bf16 buffer
    with pytest.raises(ValueError, match="row-major"):
        B.dot(a, b, out=torch.zeros(48, 32, dtype=bf16).t())


def test_scale_vectors_are_checked():
    a, b = ab()
    with pytest.raises(TypeError, match="float32"):
        B.dot(a, b, row_scale=torch.ones(32, dtype=bf16))
    with pytest.raises(ValueError, match="32 elements"):
        B.dot(a, b, row_scale=torch.ones(31))
    with pytest.raises(ValueError, match="48 elements"):
        B.dot(a, b, col_scale=torch.ones(96)[::2])                            # right length, not contiguous
    with pytest.raises(ValueError, match="48 elements"):
        B.dot(a, b, col_scale=torch.ones(48, 1))


def test_cpu_tensors_are_refused_not_computed():
    a, b = ab()
    with pytest.raises(ValueError, match="no CPU path"):
        B.dot(a, b)


def test_plan_buffer_check_without_a_device():
    """DotPlan.run's check of the buffers against the plan's problem, on a plan object that owns no device state."""
    plan = B.DotPlan.__new__(B.DotPlan)
    plan.problem = B.make_problem(32, 48, 64, bf16, bf16, row_scale=True)
    a, b = ab()
    with pytest.raises(ValueError, match="CUDA tensors on one device"):
        plan._check_buffers(a, b, torch.zeros(32, 48, dtype=bf16), torch.ones(32), None)
    assert B._span_elements(torch.zeros(32, 48)[:, :40]) == 31 * 48 + 40
    assert B._span_elements(torch.zeros(0, 48)) == 0
    plan._h = None
