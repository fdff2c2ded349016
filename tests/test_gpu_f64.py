"""f64 instances of the operator surface against the CPU oracle."""
import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import linalg, nn
from oracle import ref

pytestmark = pytest.mark.gpu
f64 = np.float64


def T(a):
    return linalg.Tensor(a, dtype="f64")


@pytest.mark.parametrize("n", [1, 2, 3, 7, 1025, 100003, (1 << 21) + 1])
def test_ring_ops_and_relu_are_bit_exact(n):
    rng = np.random.default_rng(n)
    a, b = rng.uniform(-4, 4, n), rng.uniform(1, 4, n)
    ta, tb = T(a), T(b)
    for name, got in (("add", ta + tb), ("sub", ta - tb), ("mul", ta * tb), ("div", ta / tb)):
        assert np.array_equal(got.numpy(), ref.binary64(name, a, b)), name
    assert np.array_equal((-ta).numpy(), -a)
    assert np.array_equal(nn.relu(ta).numpy(), ref.unary64("relu", a))
    assert (ta + tb).dtype == "f64" and (ta + tb).numpy().dtype == f64


@pytest.mark.parametrize("n", [5, 4096, 100003])
def test_transcendentals_within_a_few_ulp(n):
    x = np.random.default_rng(n).uniform(-8, 8, n)
    t = T(x)
    for name in ("sigmoid", "tanh", "exp"):
        got, want = getattr(nn, name)(t).numpy(), ref.unary64(name, x)
        assert np.max(np.abs(got - want) / np.abs(want)) <= 1e-14, name


def test_relu_edge_values():
    x = np.array([np.nan, -0.0, 0.0, -1.0, np.inf, -np.inf])
    r = nn.relu(T(x)).numpy()
    assert np.isnan(r[0]) and not np.signbit(r[1]) and r[4] == np.inf and r[5] == 0


@pytest.mark.parametrize("n", [1, 2, 33, 4096, 100003, (1 << 21) + 3])
def test_sum_mean_max(n):
    v = np.random.default_rng(n).standard_normal(n)
    t = T(v)
    scale = np.abs(v).sum()
    assert abs(nn.sum(t) - ref.reduce64("sum", v)) <= 1e-14 * scale
    assert abs(nn.mean(t) - ref.reduce64("mean", v)) <= 1e-14 * scale / n
    assert nn.max_of(t) == ref.reduce64("max", v)
    assert np.isnan(nn.max_of(T(np.array([np.nan, 5.0])))) and nn.max_of(T(np.array([2.0, np.nan, 3.0]))) == 3.0


@pytest.mark.parametrize("m,n,k", [(2, 2, 3), (33, 65, 17), (100, 130, 77), (256, 256, 256)])
def test_matmul_is_bit_identical_to_the_reference_loop(m, n, k):
    rng = np.random.default_rng(m * n * k)
    a, b = rng.uniform(-1, 1, (m, k)), rng.uniform(-1, 1, (k, n))
    assert np.array_equal(linalg.matmul(T(a), T(b)).numpy(), ref.matmul64(a, b))


def test_known_answers_and_fill_and_index():
    c = linalg.matmul(T([[1, 2, 3], [4, 5, 6]]), T([[7, 8], [9, 10], [11, 12]]))
    assert (c[0, 0], c[0, 1], c[1, 0], c[1, 1]) == (58.0, 64.0, 139.0, 154.0)
    assert not linalg.Tensor.zero(3, 5, dtype="f64").numpy().any()
    assert linalg.Tensor.filled(7.0, 2, 2, 2, dtype="f64")[1, 1, 1] == 7.0
    v = T([1.0, 5.0, 3.0])
    assert nn.sum(v) == 9.0 and nn.mean(v) == 3.0 and nn.max_of(v) == 5.0
    assert nn.sigmoid(T([0.0]))[0] == 0.5 and nn.tanh(T([0.0]))[0] == 0.0


def test_element_types_do_not_mix():
    a32, a64 = linalg.Tensor(np.ones(4, np.float32)), T(np.ones(4))
    with pytest.raises(TypeError):
        a32 + a64
    with pytest.raises(TypeError):
        linalg.matmul(linalg.Tensor(np.ones((2, 2), np.float32)), T(np.ones((2, 2))))
    L = cb.lib()
    assert L.cleave_cuda_add_f32(a32._h, a64._h) is None and L.cleave_cuda_last_error() == 4
    assert b"f64" in L.cleave_cuda_last_error_message()
    L.cleave_cuda_clear_error()
