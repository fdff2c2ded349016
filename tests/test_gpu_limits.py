"""Edge cases at the ends of the size range: empty inputs are refused, the largest tensor a
cleave shape can describe (2^31 - 1 elements, i32 dims) goes through the streaming and reduction
kernels, and the largest benchmark GEMM is checked through a size-independent property."""
import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import linalg, nn, workloads

pytestmark = pytest.mark.gpu
f32 = np.float32


def test_empty_tensors_are_refused():
    L = cb.lib()
    assert L.cleave_cuda_alloc_f32(0) is None and L.cleave_cuda_last_error() == 4
    assert L.cleave_cuda_zeros_f32(-5) is None
    assert L.cleave_cuda_alloc_f64(0) is None
    L.cleave_cuda_clear_error()
    with pytest.raises(TypeError):
        linalg.Tensor(np.zeros((0, 3), f32))
    a = linalg.Tensor(np.ones((2, 2), f32))
    assert L.cleave_cuda_gemm_f32(a._h, a._h, 2, 2, 0) is None     # k = 0: no empty contraction in cleave
    L.cleave_cuda_clear_error()


def test_largest_describable_tensor():
    n = (1 << 31) - 1                      # 8 GiB of f32
    ones = linalg.Tensor.filled(1.0, n)
    assert abs(nn.sum(ones) - float(1 << 31)) <= 1e-6 * (1 << 31)   # the tree's partial sums round above 2^24
    assert nn.mean(ones) == 1.0
    assert nn.max_of(ones) == 1.0
    twos = ones + ones
    assert twos[0] == 2.0 and twos[n - 1] == 2.0 and twos[n // 2 + 1] == 2.0
    assert abs(nn.sum(twos) - float(1 << 32)) <= 1e-6 * (1 << 32)
    neg = -twos
    del twos
    assert nn.max_of(neg) == -2.0 and nn.sum(nn.relu(neg)) == 0.0


def test_gemm_16384_cubed_identity_property():
    # C = I * B must reproduce B (3xTF32: hi + lo carry 22 of B's 24 significand bits);
    # any tile-scheduling, descriptor or epilogue error at this size shows as a mismatch.
    n = 16384
    b = workloads.uniform_pm1(77, n, n)
    tb = linalg.Tensor(b)
    I = np.zeros((n, n), f32)
    I[np.arange(n), np.arange(n)] = 1.0
    c = linalg.Tensor.empty(n, n)
    linalg.gemm_into(c, linalg.Tensor(I), tb, algo=linalg.GEMM_3XTF32)
    got = c.numpy()
    assert np.max(np.abs(got - b)) <= 2e-6
    # and B * I, which exercises the transposing operand pre-pass at full size
    linalg.gemm_into(c, tb, linalg.Tensor(I), algo=linalg.GEMM_3XTF32)
    assert np.max(np.abs(c.numpy() - b)) <= 2e-6
