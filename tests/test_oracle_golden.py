"""Pins the CPU oracle to every known-answer vector the reference holds for the tensor path.

The vectors live in tests/golden/reference_kats.json (transcribed from the reference's own
tests and examples, each with its source citation).  'exact' comparisons use == on float32,
as the reference's compiled test programs do.
"""
import json
import os

import numpy as np

from oracle import ref

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_kats.json")) as f:
    KATS = json.load(f)

f32 = np.float32


def test_matmul_known_answers_exact():
    for case in KATS["matmul"]:
        a, b, c = (np.array(case[k], f32) for k in ("a", "b", "c"))
        assert np.array_equal(ref.matmul(a, b), c), case["cite"]
        assert np.array_equal(ref.matmul(a, b, faithful_loop_order=True), c), case["cite"]


def test_add_known_answers_exact():
    for case in KATS["add"]:
        a, b, c = (np.array(case[k], f32) for k in ("a", "b", "c"))
        assert np.array_equal(ref.add(a, b), c), case["cite"]


def test_index_is_row_major():
    # tensor.extract on a row-major dense tensor (mlir_lower.rs:1972-2002)
    for case in KATS["index"]:
        data = np.array(case["data"], f32)
        assert data[tuple(case["idx"])] == f32(case["value"]), case["cite"]
        flat = np.ravel_multi_index(tuple(case["idx"]), data.shape)
        assert data.ravel()[flat] == f32(case["value"])


def test_activation_known_answers_exact():
    for case in KATS["activation"]:
        x, y = np.array(case["x"], f32), np.array(case["y"], f32)
        got = getattr(ref, case["op"])(x)
        assert np.array_equal(got, y), case
        assert not np.signbit(got[y == 0]).any()  # relu(-2) is +0, tanh(0) is +0


def test_relu_propagates_nan_and_orders_zeros():
    x = np.array([np.nan, -0.0, 0.0, -1.0, np.inf, -np.inf], f32)
    r = ref.relu(x)
    assert np.isnan(r[0])
    assert r[1] == 0 and not np.signbit(r[1])  # maximumf(-0, +0) = +0
    assert r[2] == 0 and r[3] == 0 and r[4] == np.inf and r[5] == 0


def test_reductions_known_answers_exact():
    for case in KATS["reduce"]:
        v = np.array(case["v"], f32)
        assert ref.sum(v) == f32(case["sum"])
        assert ref.mean(v) == f32(case["mean"])
        assert ref.max_of(v) == f32(case["max"])


def test_sum_is_left_to_right():
    # 1e8 + 1 - 1e8 in float32: left-to-right gives 0, any pairing of (1, -1e8) first would too,
    # but (1e8 + -1e8) + 1 gives 1: the order is observable.
    v = np.array([1e8, 1.0, -1e8], f32)
    assert ref.sum(v) == f32(0.0)
    v = np.array([1e8, -1e8, 1.0], f32)
    assert ref.sum(v) == f32(1.0)


def test_max_is_strict_scan_from_first():
    v = np.array([2.0, np.nan, 3.0, 1.0], f32)
    assert ref.max_of(v) == f32(3.0)  # NaN > acc is false, so NaN is skipped
    v = np.array([np.nan, 5.0], f32)
    assert np.isnan(ref.max_of(v))  # 5 > NaN is false, acc stays NaN


def test_derivative_known_answers():
    for case in KATS["derivative"]:
        if case["op"] == "tanh_bwd":
            x = f32(case["x"])
            t = ref.tanh(np.array([x]))[0]
            expected = f32(1.0) - t * t
            got = ref.tanh_bwd(np.array([t]), np.array([1.0], f32))[0]
            assert got == expected
        elif case["op"] == "sigmoid_sq":
            # loss = s*s; dloss/ds = 2s (as s*1 + 1*s), chained through sigmoid' = s(1-s)
            w = f32(case["x"])
            s = ref.sigmoid(np.array([w]))[0]
            expected = f32(2.0) * s * s * (f32(1.0) - s)
            got = ref.sigmoid_bwd(np.array([s]), np.array([s + s], f32))[0]
            assert abs(got - expected) <= 2 * np.spacing(expected)
        elif case["op"] == "two_sigmoids":
            s1 = ref.sigmoid(np.array([case["w1"]], f32))[0]
            s2 = ref.sigmoid(np.array([case["w2"]], f32))[0]
            g0 = ref.sigmoid_bwd(np.array([s1]), np.array([s2]))[0]
            g1 = ref.sigmoid_bwd(np.array([s2]), np.array([s1]))[0]
            assert abs(g0 - s1 * (1 - s1) * s2) < case["tol"]
            assert abs(g1 - s1 * s2 * (1 - s2)) < case["tol"]
        elif case["op"] == "matmul_identity_trace":
            # f = trace(A I); dA = dC I^T with dC = I
            dC = np.eye(2, dtype=f32)
            dA = ref.matmul_nt(dC, np.eye(2, dtype=f32))
            assert np.array_equal(dA.ravel(), np.array(case["grad"], f32))


def test_neuron_demo_forward():
    n = KATS["neuron"]
    w, x = np.array(n["weights"], f32), np.array(n["inputs"], f32)
    z = ref.sum(ref.mul(w, x)) + f32(n["bias"])
    act = ref.sigmoid(np.array([z], f32))[0]
    assert abs(float(act) - n["expected"]) <= n["tol"]


def test_xor_training_reproduces_the_documented_outputs():
    k = KATS["xor_training"]
    W1, b1, W2, b2 = (np.array(k[n], f32) for n in ("W1", "b1", "W2", "b2"))
    xs, ys = np.array(k["x"], f32), np.array(k["y"], f32)
    lr = f32(k["lr"])
    for step in range(k["steps"]):
        i = step % 4
        r = ref.mlp2_fwd_bwd(xs[i:i + 1], W1, b1, W2, b2, ys[i:i + 1].reshape(1, 1),
                             act1="sigmoid", act2="sigmoid", mean_loss=False)
        W1, b1 = ref.sgd(W1, r["dW1"], lr), ref.sgd(b1, r["db1"], lr)
        W2, b2 = ref.sgd(W2, r["dW2"], lr), ref.sgd(b2, r["db2"], lr)
    zero = np.zeros((4, 1), f32)
    out = ref.mlp2_fwd_bwd(xs, W1, b1, W2, b2, zero, act1="sigmoid", act2="sigmoid")["Y"].ravel()
    assert np.allclose(out, np.array(k["expected"], f32), rtol=0, atol=k["tol"]), out


def test_linear_regression_example_descends():
    k = KATS["linear_regression"]
    X = np.stack([np.array(k["xs"], f32), np.ones(4, f32)], axis=1)  # columns: x, 1 -> params (w, b)
    y = np.array(k["ys"], f32)
    p = np.zeros(2, f32)
    losses = []
    for _ in range(k["steps"]):
        loss, _, g = ref.linreg_step(X, y, p)
        # the example's loss is the SUM of squares: mean * 4
        losses.append(float(loss) * 4)
        p = ref.sgd(p, g * f32(4.0), k["lr"])
    assert losses[0] == 164.0  # 9 + 25 + 49 + 81 at w = b = 0
    assert all(b < a for a, b in zip(losses, losses[1:]))
    loss64, g64 = ref.linreg_step_f64(X, y, p)
    loss32, _, g32 = ref.linreg_step(X, y, p)
    assert abs(loss64 - float(loss32)) <= 1e-5 * loss64
    assert np.allclose(g64, g32, rtol=1e-5)


def test_loop_orders_agree_bit_for_bit():
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (37, 129)).astype(f32)
    b = rng.uniform(-1, 1, (129, 53)).astype(f32)
    c = ref.matmul(a, b)
    assert np.array_equal(c, ref.matmul(a, b, faithful_loop_order=True))
    assert np.array_equal(c[5:9], ref.matmul_rows(a, b, 5, 4))
    assert np.array_equal(ref.matmul_tn(np.ascontiguousarray(a.T), b), c)
    assert np.array_equal(ref.matmul_nt(a, np.ascontiguousarray(b.T)), c)
    c64 = ref.matmul_f64(a, b)
    s = ref.matmul_absdot(a, b)
    assert np.max(np.abs(c - c64) / s) < 1e-6


def test_mlp2_gradients_match_finite_differences():
    rng = np.random.default_rng(1)
    X = rng.standard_normal((6, 5)).astype(f32)
    W1 = (rng.standard_normal((5, 7)) * 0.3).astype(f32)
    b1 = (rng.standard_normal(7) * 0.1).astype(f32)
    W2 = (rng.standard_normal((7, 3)) * 0.3).astype(f32)
    b2 = (rng.standard_normal(3) * 0.1).astype(f32)
    T = rng.uniform(0, 1, (6, 3)).astype(f32)

    def loss64(W1, b1, W2, b2):
        H = np.tanh(X.astype(np.float64) @ W1 + b1)
        Y = 1 / (1 + np.exp(-(H @ W2 + b2)))
        return np.mean((Y - T) ** 2)

    r = ref.mlp2_fwd_bwd(X, W1, b1, W2, b2, T)
    eps = 1e-6
    P = [a.astype(np.float64) for a in (W1, b1, W2, b2)]
    for pi, name in enumerate(("dW1", "db1", "dW2", "db2")):
        g = np.zeros_like(P[pi])
        it = np.nditer(P[pi], flags=["multi_index"])
        for _ in it:
            idx = it.multi_index
            Pp = [p.copy() for p in P]
            Pm = [p.copy() for p in P]
            Pp[pi][idx] += eps
            Pm[pi][idx] -= eps
            g[idx] = (loss64(*Pp) - loss64(*Pm)) / (2 * eps)
        assert np.allclose(r[name], g, rtol=1e-3, atol=1e-6), name
