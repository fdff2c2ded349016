"""Parity of the streaming operators with the CPU oracle, through the C ABI."""
import json
import os

import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import linalg, nn
from oracle import ref

from _util import TOL, rel_err

pytestmark = pytest.mark.gpu
f32 = np.float32
SIZES = [1, 3, 4, 7, 33, 127, 129, 1024, 4097, 1 << 20, (1 << 22) + 5]


def rnd(seed, n, lo=-4.0, hi=4.0):
    return np.random.default_rng(seed).uniform(lo, hi, n).astype(f32)


@pytest.mark.parametrize("n", SIZES)
def test_ring_ops_are_bit_exact(n):
    a, b = rnd(1, n), rnd(2, n)
    b[np.abs(b) < 1e-3] = 1.0
    ta, tb = linalg.Tensor(a), linalg.Tensor(b)
    assert np.array_equal((ta + tb).numpy(), ref.add(a, b))
    assert np.array_equal((ta - tb).numpy(), ref.sub(a, b))
    assert np.array_equal((ta * tb).numpy(), ref.mul(a, b))
    assert np.array_equal((ta / tb).numpy(), ref.div(a, b))
    assert np.array_equal((-ta).numpy(), ref.neg(a))


def test_ring_ops_on_rank_2_and_3_and_special_values():
    a = np.array([[np.inf, -np.inf, np.nan], [0.0, -0.0, 1e-45]], f32)
    b = np.array([[1.0, np.inf, 2.0], [0.0, 5.0, 1e38]], f32)
    with np.errstate(all="ignore"):
        for got, want in (((linalg.Tensor(a) + linalg.Tensor(b)).numpy(), ref.add(a, b)),
                          ((linalg.Tensor(a) * linalg.Tensor(b)).numpy(), ref.mul(a, b)),
                          ((linalg.Tensor(a) / linalg.Tensor(b)).numpy(), ref.div(a, b))):
            assert np.array_equal(got, want, equal_nan=True)
            ok = ~np.isnan(want)   # the sign of a generated NaN is not specified by IEEE 754
            assert np.array_equal(np.signbit(got[ok]), np.signbit(want[ok]))
    t3 = linalg.Tensor(np.arange(8, dtype=f32).reshape(2, 2, 2) + 1)
    assert t3[0, 1, 0] == 3.0 and t3[1, 1, 1] == 8.0


@pytest.mark.parametrize("n", SIZES)
def test_relu_is_bit_exact_and_transcendentals_within_tolerance(n):
    x = rnd(3, n, -10, 10)
    t = linalg.Tensor(x)
    assert np.array_equal(nn.relu(t).numpy(), ref.relu(x))
    assert rel_err(nn.sigmoid(t).numpy(), ref.sigmoid(x)) <= TOL
    assert rel_err(nn.tanh(t).numpy(), ref.tanh(x)) <= TOL
    assert rel_err(nn.exp(t).numpy(), ref.exp(x)) <= TOL


def test_activation_edge_values():
    x = np.array([np.nan, -0.0, 0.0, -np.inf, np.inf, -100.0, 100.0, 1e-30], f32)
    t = linalg.Tensor(x)
    r = nn.relu(t).numpy()
    assert np.array_equal(r, ref.relu(x), equal_nan=True) and not np.signbit(r[1])
    with np.errstate(all="ignore"):
        assert np.allclose(nn.sigmoid(t).numpy(), ref.sigmoid(x), rtol=TOL, atol=0, equal_nan=True)
        assert np.allclose(nn.tanh(t).numpy(), ref.tanh(x), rtol=TOL, atol=0, equal_nan=True)


@pytest.mark.parametrize("n", [5, 1024, 100003])
def test_derivative_forms_are_bit_exact(n):
    y = rnd(4, n, -1, 1)
    g = rnd(5, n)
    ty, tg = linalg.Tensor(y), linalg.Tensor(g)
    assert np.array_equal(nn.tanh_bwd(ty, tg).numpy(), ref.tanh_bwd(y, g))
    assert np.array_equal(nn.sigmoid_bwd(ty, tg).numpy(), ref.sigmoid_bwd(y, g))
    assert np.array_equal(nn.relu_bwd(ty, tg).numpy(), ref.relu_bwd(y, g))


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (17, 64), (129, 1024), (1000, 33)])
@pytest.mark.parametrize("act", ["identity", "relu", "sigmoid", "tanh"])
def test_bias_act(rows, cols, act):
    x = rnd(6, rows * cols).reshape(rows, cols)
    b = rnd(7, cols)
    want = ref.bias_add(x, b)
    if act != "identity":
        want = getattr(ref, act)(want)
    got = nn.bias_act(linalg.Tensor(x), linalg.Tensor(b), act).numpy()
    if act in ("identity", "relu"):
        assert np.array_equal(got, want)
    else:
        assert rel_err(got, want) <= TOL


def test_sgd_update_in_place_is_bit_exact():
    w, g = rnd(8, 100003), rnd(9, 100003)
    tw, tg = linalg.Tensor(w), linalg.Tensor(g)
    nn.sgd_step(tw, tg, 1e-3)
    assert np.array_equal(tw.numpy(), ref.sgd(w, g, 1e-3))
    nn.sgd_step(tw, tg, 0.5, gscale=0.125)   # exact power-of-two scale
    assert np.array_equal(tw.numpy(), ref.sgd(ref.sgd(w, g, 1e-3), g * f32(0.125), 0.5))


def test_fill_zero_and_index():
    z = linalg.Tensor.zero(3, 5)
    assert not z.numpy().any()
    for dims in ((3,), (2, 2), (2, 2, 2)):
        t = linalg.Tensor.filled(7.0, *dims)
        assert t[tuple(0 for _ in dims)] == 7.0 and t[tuple(d - 1 for d in dims)] == 7.0
    big = linalg.Tensor.filled(-1.5, 1 << 20)
    assert (big.numpy() == f32(-1.5)).all()


def test_unaligned_views_take_the_scalar_path():
    a, b = rnd(10, 1001), rnd(11, 1001)
    ta, tb = linalg.Tensor(a), linalg.Tensor(b)
    va = linalg.Tensor.from_device_ptr(ta.data_ptr + 4, 1000)
    vb = linalg.Tensor.from_device_ptr(tb.data_ptr + 4, 1000)
    assert np.array_equal((va + vb).numpy(), a[1:] + b[1:])
    assert np.array_equal(nn.relu(va).numpy(), ref.relu(a[1:]))


def test_reference_known_answers_through_the_c_abi():
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")) as f:
        kats = json.load(f)
    for case in kats["add"]:
        got = (linalg.Tensor(case["a"]) + linalg.Tensor(case["b"])).numpy()
        assert np.array_equal(got, np.array(case["c"], f32)), case["cite"]
    for case in kats["activation"]:
        got = getattr(nn, case["op"])(linalg.Tensor(case["x"])).numpy()
        assert np.array_equal(got, np.array(case["y"], f32)), case
    for case in kats["index"]:
        assert linalg.Tensor(case["data"])[tuple(case["idx"])] == case["value"]
    for case in kats["reduce"]:
        v = linalg.Tensor(case["v"])
        assert nn.sum(v) == case["sum"] and nn.mean(v) == case["mean"] and nn.max_of(v) == case["max"]
    n = kats["neuron"]
    z = nn.sum(linalg.Tensor(n["weights"]) * linalg.Tensor(n["inputs"])) + f32(n["bias"])
    act = nn.sigmoid(linalg.Tensor([z]))[0]
    assert abs(act - n["expected"]) <= n["tol"]


def test_errors_are_reported_not_swallowed():
    a = linalg.Tensor(rnd(1, 8))
    L = cb.lib()
    assert L.cleave_cuda_add_f32(a._h, linalg.Tensor(rnd(2, 9))._h) is None
    assert L.cleave_cuda_last_error() == 3   # shape
    L.cleave_cuda_clear_error()
    h = L.cleave_cuda_alloc_f32(4)
    L.cleave_cuda_free(h)
    assert L.cleave_cuda_len(h) == -2        # freed handle is no longer live
    L.cleave_cuda_clear_error()
