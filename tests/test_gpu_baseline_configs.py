"""Parity at the benchmark configurations themselves, each through the route the library picks there.

The oracle's scalar loop cannot finish the whole of an 8192^3 product inside a test, so the large
products are checked on sampled rows computed exactly as the reference loop computes them
(stdlib/linalg/matrix.cleave:59-60, cleave/src/mlir_lower.rs:2089-2120: zero-initialised accumulator,
multiply then add, k ascending) plus the linearity checksum (1^T A) B = 1^T (A B) over the whole result.
The two-layer perceptron of configuration 2 is small enough for a full oracle pass (~90 GMAC).
"""
import os

import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import autodiff, linalg, workloads
from cleave_b200.linalg import GEMM_AUTO, GEMM_3XTF32
from oracle import ref

from _util import TOL, assert_gemm_close

pytestmark = pytest.mark.gpu
f32 = np.float32


def _sampled_rows(m, count, seed):
    return np.concatenate([np.sort(np.random.default_rng(seed).choice(m - 8, count, replace=False)),
                           np.arange(m - 8, m)])


def _linearity(got, a, b):
    lhs = a.astype(np.float64).sum(axis=0) @ b.astype(np.float64)
    rhs = got.astype(np.float64).sum(axis=0)
    scale = np.abs(a).astype(np.float64).sum(axis=0) @ np.abs(b).astype(np.float64)
    return float(np.max(np.abs(lhs - rhs) / scale))


def _product(a, b, algo):
    c = linalg.Tensor.empty(a.shape[0], b.shape[1])
    L = cb.lib()
    before = L.cleave_cuda_kernel_launches()
    linalg.gemm_into(c, linalg.Tensor(a), linalg.Tensor(b), algo=algo)
    cb.sync()
    return c.numpy(), L.cleave_cuda_kernel_launches() - before


def test_headline_8192_cubed_default_route_sampled_rows():
    # The headline workload: two split pre-passes + the CTA-pair kernel, K = 8192 = 32 accumulator restarts.
    m = n = k = 8192
    a, b = workloads.gemm_inputs(m, n, k)
    got, launches = _product(a, b, GEMM_3XTF32)
    assert launches == 3
    rows = _sampled_rows(m, 64, 8192)
    e = assert_gemm_close(np.ascontiguousarray(got[rows]), np.ascontiguousarray(a[rows]), b, what="8192^3 sampled rows")
    print("8192^3 errors:", e)
    assert _linearity(got, a, b) <= TOL
    # the dispatcher's own choice must be the same route and the same bits
    auto, _ = _product(a, b, GEMM_AUTO)
    assert np.array_equal(auto, got)


@pytest.mark.parametrize("m,n,k", [(16384, 16384, 64), (16384, 64, 16384)])
def test_skinny_sweep_shapes_at_size(m, n, k):
    a, b = workloads.gemm_inputs(m, n, k)
    got, _ = _product(a, b, GEMM_AUTO)
    rows = _sampled_rows(m, 56, m + n)
    assert_gemm_close(np.ascontiguousarray(got[rows]), np.ascontiguousarray(a[rows]), b, what=("skinny", m, n, k))
    assert _linearity(got, a, b) <= TOL


@pytest.mark.parametrize("size", [1024, 2048])
def test_small_square_sweep_shapes_full_oracle(size):
    a, b = workloads.gemm_inputs(size, size, size)
    got, _ = _product(a, b, GEMM_AUTO)
    assert_gemm_close(got, a, b, what=("square", size))


def test_batched_4096_cubed_entries_on_both_sides_of_a_workspace_chunk():
    # 34 independent 4096^3 products in one call: the operand workspace is bounded, so the batch is processed in
    # chunks; entries of the first chunk, the entries either side of the chunk border and the last one are checked.
    batch, sz = 34, 4096
    A = np.empty((batch, sz, sz), f32)
    B = np.empty((batch, sz, sz), f32)
    for i in range(batch):
        A[i] = workloads.uniform_pm1(100 + i, sz, sz)
        B[i] = workloads.uniform_pm1(300 + i, sz, sz)
    ta, tb = linalg.Tensor(A), linalg.Tensor(B)
    tc = linalg.Tensor.empty(batch, sz, sz)
    linalg.gemm_into(tc, ta, tb)
    cb.sync()
    rows = _sampled_rows(sz, 8, 34)
    for i in (0, 17, 31, 32, 33):
        entry = linalg.Tensor.from_device_ptr(tc.data_ptr + 4 * i * sz * sz, sz, sz)
        got = entry.numpy()
        assert_gemm_close(np.ascontiguousarray(got[rows]), np.ascontiguousarray(A[i][rows]), B[i], what=("batch entry", i))
        assert _linearity(got, A[i], B[i]) <= TOL


def test_batch_chunking_with_a_small_workspace_limit():
    # The same chunk loop on every operand route, with the workspace limit lowered so that a small batch crosses it.
    os.environ["CLEAVE_CUDA_GEMM_WORKSPACE_MB"] = "1"
    try:
        for (batch, m, n, k) in [(7, 256, 512, 128), (5, 260, 300, 100), (6, 384, 256, 512)]:
            A = workloads.uniform_pm1(21, batch, m, k)
            B = workloads.uniform_pm1(22, batch, k, n)
            tc = linalg.Tensor.empty(batch, m, n)
            linalg.gemm_into(tc, linalg.Tensor(A), linalg.Tensor(B), algo=GEMM_3XTF32)
            cb.sync()
            got = tc.numpy()
            for i in range(batch):
                assert_gemm_close(got[i], A[i], B[i], what=("chunked", batch, m, n, k, i))
    finally:
        del os.environ["CLEAVE_CUDA_GEMM_WORKSPACE_MB"]


def test_mlp_config_2_at_full_size():
    # batch 4096, 1024 -> 4096 (tanh) -> 1024 (sigmoid), MSE; every gradient against the oracle's full pass.
    X, W1, b1, W2, b2, T = workloads.mlp_inputs()
    want = ref.mlp2_fwd_bwd(X, W1, b1, W2, b2, T)
    net = autodiff.MLP2(1024, 4096, 1024)
    net.load(W1, b1, W2, b2)
    loss = net.forward_backward(linalg.Tensor(X), linalg.Tensor(T))
    cb.sync()
    loss64 = ref.mse_f64(want["Y"], T)
    assert abs(loss - loss64) <= TOL * loss64
    absX, absH = np.abs(X).astype(np.float64), np.abs(want["H"]).astype(np.float64)
    adZ2, adZ1 = np.abs(want["dZ2"]).astype(np.float64), np.abs(want["dZ1"]).astype(np.float64)

    def check(got, ref32, scale, what):
        err = float(np.max(np.abs(got.astype(np.float64) - ref32) / np.maximum(scale, 1e-30)))
        assert err <= TOL, (what, err)

    check(net.dW2.numpy(), want["dW2"], absH.T @ adZ2, "dW2")
    check(net.db2.numpy(), want["db2"], adZ2.sum(axis=0), "db2")
    check(net.dW1.numpy(), want["dW1"], absX.T @ adZ1, "dW1")
    check(net.db1.numpy(), want["db1"], adZ1.sum(axis=0), "db1")
    # forward values, from a pass that keeps them
    _, inter = net.forward_backward(linalg.Tensor(X), linalg.Tensor(T), keep=True)
    cb.sync()
    check(inter["H"].numpy(), want["H"], absX @ np.abs(W1).astype(np.float64) + np.abs(b1), "H")
    check(inter["Y"].numpy(), want["Y"], absH @ np.abs(W2).astype(np.float64) + np.abs(b2), "Y")
    check(inter["dZ1"].numpy(), want["dZ1"], adZ2 @ np.abs(W2).astype(np.float64).T, "dZ1")


def test_linreg_config_1_at_full_size():
    # 1,048,576 x 16 with the configuration's own seeded data (y = X w* + noise): pred bit for bit, loss and
    # gradient against the f64 evaluation.
    X, y, _ = workloads.linreg_inputs()
    w = workloads.normal(70, 16) * f32(0.5)
    loss, grad, pred = autodiff.linreg_step(linalg.Tensor(X), linalg.Tensor(y), linalg.Tensor(w))
    _want_loss, want_pred, _want_grad = ref.linreg_step(X, y, w)
    assert np.array_equal(pred.numpy(), want_pred)
    loss64, grad64 = ref.linreg_step_f64(X, y, w)
    assert abs(loss - loss64) <= TOL * loss64
    e = np.abs(want_pred.astype(np.float64) - y)
    scale = (2.0 / X.shape[0]) * (np.abs(X).astype(np.float64) * e[:, None]).sum(axis=0)
    assert np.max(np.abs(grad.numpy() - grad64) / scale) <= TOL
