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


def _wrap(handle, *dims):
    assert handle, cb.lib().cleave_cuda_last_error_message()
    return linalg.Tensor._wrap(handle, dims, "f64 op", "f64")


def test_derivative_forms_and_sgd_are_bit_exact():
    # (1 - y*y) * g, y*(1 - y) * g, x > 0 ? g : 0, w - lr*(gscale*g): one rounded operation per step, as the
    # separate arith ops of the lowered program (stdlib/num/num.cleave:123-136, :222-223)
    L = cb.lib()
    rng = np.random.default_rng(3)
    n = 100003
    y, g = rng.uniform(-1, 1, n), rng.standard_normal(n)
    ty, tg = T(y), T(g)
    one = np.ones(n)
    want = ref.binary64("mul", ref.binary64("sub", one, ref.binary64("mul", y, y)), g)
    assert np.array_equal(_wrap(L.cleave_cuda_tanh_bwd_f64(ty._h, tg._h), n).numpy(), want)
    want = ref.binary64("mul", ref.binary64("mul", y, ref.binary64("sub", one, y)), g)
    assert np.array_equal(_wrap(L.cleave_cuda_sigmoid_bwd_f64(ty._h, tg._h), n).numpy(), want)
    assert np.array_equal(_wrap(L.cleave_cuda_relu_bwd_f64(ty._h, tg._h), n).numpy(), np.where(y > 0, g, 0.0))
    w = rng.standard_normal(n)
    tw = T(w)
    assert L.cleave_cuda_sgd_f64(tw._h, tg._h, 0.1, 0.25) == 0
    want = ref.binary64("sub", w, ref.binary64("mul", np.full(n, 0.1), ref.binary64("mul", np.full(n, 0.25), g)))
    assert np.array_equal(tw.numpy(), want)


@pytest.mark.parametrize("m,n,k", [(33, 65, 17), (100, 130, 77), (128, 64, 256)])
def test_transposed_and_batched_matmul_are_bit_identical_to_the_reference_loop(m, n, k):
    L = cb.lib()
    rng = np.random.default_rng(m + n + k)
    a, b = rng.uniform(-1, 1, (m, k)), rng.uniform(-1, 1, (k, n))
    want = ref.matmul64(a, b)
    ta, tb, at, bt = T(a), T(b), T(np.ascontiguousarray(a.T)), T(np.ascontiguousarray(b.T))   # keep the handles alive
    assert np.array_equal(_wrap(L.cleave_cuda_gemm_tn_f64(at._h, tb._h, m, n, k), m, n).numpy(), want)
    assert np.array_equal(_wrap(L.cleave_cuda_gemm_nt_f64(ta._h, bt._h, m, n, k), m, n).numpy(), want)
    A, B = rng.uniform(-1, 1, (3, m, k)), rng.uniform(-1, 1, (3, k, n))
    tA, tB = T(A), T(B)
    got = _wrap(L.cleave_cuda_gemm_batched_f64(tA._h, tB._h, 3, m, n, k), 3, m, n).numpy()
    for i in range(3):
        assert np.array_equal(got[i], ref.matmul64(A[i], B[i]))


def test_colsum_and_mse():
    L = cb.lib()
    rng = np.random.default_rng(9)
    x = rng.standard_normal((1000, 333))
    tx = T(x)
    got = _wrap(L.cleave_cuda_colsum_f64(tx._h, 1000, 333), 333).numpy()
    assert np.max(np.abs(got - x.sum(axis=0)) / np.abs(x).sum(axis=0)) <= 1e-14
    p, t = rng.uniform(0, 1, 100003), rng.uniform(0, 1, 100003)
    d = linalg.Tensor.zero(100003, dtype="f64")
    tp, tt, short = T(p), T(t), T(t[:5])
    loss = L.cleave_cuda_mse_f64(tp._h, tt._h, d._h)
    e = ref.binary64("sub", p, t)
    assert abs(loss - np.mean(e * e)) <= 1e-14 * np.mean(e * e)
    want_d = ref.binary64("div", ref.binary64("mul", np.full(p.size, 2.0), e), np.full(p.size, float(p.size)))
    assert np.array_equal(d.numpy(), want_d)
    assert np.isnan(L.cleave_cuda_mse_f64(tp._h, short._h, None))
    assert L.cleave_cuda_last_error() == 3
    L.cleave_cuda_clear_error()
