"""Parity of reductions, column sums, MSE and the linear-regression step with the CPU oracle."""
import numpy as np
import pytest

from cleave_b200 import autodiff, linalg, nn, workloads
from oracle import ref

from _util import TOL, scaled_err

pytestmark = pytest.mark.gpu
f32 = np.float32
SIZES = [1, 2, 7, 33, 255, 4096, 4097, 100003, 1 << 20, (1 << 22) + 3]


@pytest.mark.parametrize("n", SIZES)
def test_sum_mean_max(n):
    v = np.random.default_rng(n).standard_normal(n).astype(f32)
    t = linalg.Tensor(v)
    scale = ref.sum_abs_f64(v)
    # Error of a float32 summation is proportional to the sum of |terms|: both the oracle's
    # left-to-right chain and the device tree are compared on that scale, and with float64.
    assert scaled_err(nn.sum(t), ref.sum(v), scale) <= TOL
    assert scaled_err(nn.sum(t), ref.sum_f64(v), scale) <= max(scaled_err(ref.sum(v), ref.sum_f64(v), scale), 1e-7)
    assert scaled_err(nn.mean(t), ref.mean(v), scale / n) <= TOL
    assert nn.max_of(t) == ref.max_of(v)
    assert nn.sum(t) == nn.sum(t)   # reproducible


def test_sum_of_exact_values_is_exact():
    v = np.arange(1, 10001, dtype=f32)
    assert nn.sum(linalg.Tensor(v)) == 50005000.0
    assert nn.mean(linalg.Tensor(np.full(4096, 3.0, f32))) == 3.0


def test_max_nan_semantics_follow_the_strict_scan():
    assert nn.max_of(linalg.Tensor(np.array([2.0, np.nan, 3.0, 1.0], f32))) == 3.0
    assert np.isnan(nn.max_of(linalg.Tensor(np.array([np.nan, 5.0], f32))))
    assert nn.max_of(linalg.Tensor(np.array([-np.inf, -np.inf], f32))) == -np.inf
    v = np.full(100000, -5.0, f32)
    v[77777] = 9.0
    assert nn.max_of(linalg.Tensor(v)) == 9.0


@pytest.mark.parametrize("rows,cols", [(1, 1), (5, 3), (64, 128), (1000, 130), (4096, 1024), (333, 4096)])
def test_colsum(rows, cols):
    x = np.random.default_rng(rows * cols).standard_normal((rows, cols)).astype(f32)
    got = nn.colsum(linalg.Tensor(x)).numpy()
    want = ref.colsum(x)
    scale = np.abs(x).astype(np.float64).sum(axis=0)
    assert np.max(np.abs(got.astype(np.float64) - want) / scale) <= TOL
    exact = x.astype(np.float64).sum(axis=0)
    assert np.max(np.abs(got - exact) / scale) <= max(np.max(np.abs(want - exact) / scale), 1e-7)


@pytest.mark.parametrize("n", [1, 5, 4096, 100003, 1 << 22])
def test_mse_loss_and_gradient(n):
    rng = np.random.default_rng(n)
    p = rng.uniform(0, 1, n).astype(f32)
    t = rng.uniform(0, 1, n).astype(f32)
    loss, dp = nn.mse(linalg.Tensor(p), linalg.Tensor(t))
    want_loss, want_dp = ref.mse(p, t)
    assert np.array_equal(dp.numpy(), want_dp)                 # elementwise: bit-exact
    loss64 = ref.mse_f64(p, t)
    assert abs(loss - loss64) <= TOL * loss64
    # The reference's left-to-right float32 chain drifts from the exact sum as n grows (4e-3
    # relative at n = 4M); the device tree may differ from it by that drift, not by more.
    assert abs(loss - float(want_loss)) <= abs(float(want_loss) - loss64) + TOL * loss64


@pytest.mark.parametrize("rows,feat", [(1, 1), (1000, 16), (5000, 7), (4096, 32), (100003, 16), (1 << 20, 16), (777, 4), (33333, 8), (65, 32)])
def test_linreg_step(rows, feat):
    X = workloads.normal(31, rows, feat)
    w_true = workloads.normal(32, feat)
    y = (X @ w_true + workloads.normal(33, rows, sigma=0.1)).astype(f32)
    for w in (np.zeros(feat, f32), w_true):
        loss, grad, pred = autodiff.linreg_step(linalg.Tensor(X), linalg.Tensor(y), linalg.Tensor(w))
        want_loss, want_pred, want_grad = ref.linreg_step(X, y, w)
        assert np.array_equal(pred.numpy(), want_pred)          # f ascending, mul then add: bit-exact
        loss64, grad64 = ref.linreg_step_f64(X, y, w)
        assert abs(loss - loss64) <= TOL * loss64
        assert abs(loss - float(want_loss)) <= abs(float(want_loss) - loss64) + TOL * loss64
        # gradient terms X[i,f] * 2e_i/N: error scales with the sum of |terms|
        e = np.abs(want_pred.astype(np.float64) - y) * 2 / rows
        scale = np.abs(X).astype(np.float64).T @ e
        scale = np.maximum(scale, 1e-30)
        g = grad.numpy().astype(np.float64)
        assert np.max(np.abs(g - grad64) / scale) <= TOL
        # against the reference's float32 chain: allowed to differ by that chain's own drift
        # from the exact sum (3e-5 of the scale at a million rows), not by more
        drift = np.abs(want_grad - grad64) / scale
        assert np.all(np.abs(g - want_grad) / scale <= drift + TOL)


def test_linreg_step_with_the_loss_left_on_the_device():
    X = workloads.normal(31, 100003, 16)
    y = workloads.normal(33, 100003)
    w = workloads.normal(32, 16)
    tX, ty, tw = linalg.Tensor(X), linalg.Tensor(y), linalg.Tensor(w)
    loss, grad, pred = autodiff.linreg_step(tX, ty, tw)
    loss_dev, g2, p2 = linalg.Tensor.zero(1), linalg.Tensor.empty(16), linalg.Tensor.empty(100003)
    none, g, p = autodiff.linreg_step(tX, ty, tw, loss_out=loss_dev, grad_out=g2, pred_out=p2)
    assert none is None and g is g2 and p is p2
    assert loss_dev[0] == loss
    assert np.array_equal(g2.numpy(), grad.numpy()) and np.array_equal(p2.numpy(), pred.numpy())
