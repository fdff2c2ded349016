"""Forward + backward of the two-layer perceptron against the CPU oracle, stage by stage."""
import json
import os

import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import autodiff, linalg, workloads
from oracle import ref

from _util import TOL

pytestmark = pytest.mark.gpu
f32 = np.float32


def check(got, want, scale, what):
    err = np.max(np.abs(got.astype(np.float64) - want) / np.maximum(scale, 1e-30))
    assert err <= TOL, (what, err)


@pytest.mark.parametrize("batch,d_in,d_hid,d_out", [(4, 3, 5, 2), (64, 32, 48, 16), (256, 128, 512, 64),
                                                    (512, 256, 1024, 256)])
def test_mlp2_forward_backward_matches_oracle(batch, d_in, d_hid, d_out):
    X, W1, b1, W2, b2, T = workloads.mlp_inputs(batch, d_in, d_hid, d_out)
    b1 = workloads.uniform_pm1(41, d_hid) * f32(0.1)
    b2 = workloads.uniform_pm1(42, d_out) * f32(0.1)
    want = ref.mlp2_fwd_bwd(X, W1, b1, W2, b2, T)
    net = autodiff.MLP2(d_in, d_hid, d_out)
    net.load(W1, b1, W2, b2)
    loss, inter = net.forward_backward(linalg.Tensor(X), linalg.Tensor(T), keep=True)
    cb.sync()
    loss64 = ref.mse_f64(want["Y"], T)
    assert abs(loss - loss64) <= TOL * loss64
    assert abs(loss - float(want["loss"])) <= abs(float(want["loss"]) - loss64) + TOL * loss64
    # Each quantity is compared on the scale of the sum of |terms| of the contraction that made it.
    absX, absH = np.abs(X).astype(np.float64), np.abs(want["H"]).astype(np.float64)
    check(inter["H"].numpy(), want["H"], absX @ np.abs(W1) + np.abs(b1), "H")
    check(inter["Y"].numpy(), want["Y"], absH @ np.abs(W2) + np.abs(b2), "Y")
    adZ2, adZ1 = np.abs(want["dZ2"]).astype(np.float64), np.abs(want["dZ1"]).astype(np.float64)
    check(net.dW2.numpy(), want["dW2"], absH.T @ adZ2, "dW2")
    check(net.db2.numpy(), want["db2"], adZ2.sum(axis=0), "db2")
    check(inter["dH"].numpy(), want["dH"], adZ2 @ np.abs(W2).T, "dH")
    check(net.dW1.numpy(), want["dW1"], absX.T @ adZ1, "dW1")
    check(net.db1.numpy(), want["db1"], adZ1.sum(axis=0), "db1")
    # The production pass (no intermediates kept) fuses act1'(H) into the dH product's epilogue: same bits.
    kept = net.grads.numpy().copy()
    loss2 = net.forward_backward(linalg.Tensor(X), linalg.Tensor(T))
    cb.sync()
    assert loss2 == loss and np.array_equal(net.grads.numpy(), kept)


def test_xor_training_through_the_device_path():
    # examples/xor_tensor.cleave trained for 4000 SGD steps; the documented outputs are the target.
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")) as f:
        k = json.load(f)["xor_training"]
    net = autodiff.MLP2(2, 2, 1, act1="sigmoid", act2="sigmoid")
    net.load(k["W1"], k["b1"], k["W2"], k["b2"])
    xs = [linalg.Tensor(np.array([x], f32)) for x in k["x"]]
    ys = [linalg.Tensor(np.array([[y]], f32)) for y in k["y"]]
    for step in range(k["steps"]):
        i = step % 4
        net.forward_backward(xs[i], ys[i])
        net.sgd(k["lr"])     # single output: mean over one element == the example's squared error
    out = [net.forward(x)[1][0, 0] for x in xs]
    assert np.allclose(out, k["expected"], rtol=0, atol=1e-4), out


def test_sgd_training_reduces_the_loss():
    X, W1, b1, W2, b2, T = workloads.mlp_inputs(256, 64, 128, 32)
    net = autodiff.MLP2(64, 128, 32)
    net.load(W1, b1, W2, b2)
    tX, tT = linalg.Tensor(X), linalg.Tensor(T)
    losses = []
    for _ in range(20):
        losses.append(net.forward_backward(tX, tT))
        net.sgd(0.5)
    assert losses[-1] < losses[0]
