"""The chained GEMM form: lo planes handed from call to call (cleave_cuda_gemm_fused_f32, cleave_cuda_split_lo_f32,
cleave_cuda_mse_act_bwd_lo_f32).  The planes are an optimisation only: every result must be bit-identical to the
unchained entry points, and a plane written by an epilogue must equal the plane a streaming pass computes."""
import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import autodiff, linalg, nn, workloads
from cleave_b200.linalg import GEMM_AUTO, GEMM_EXACT, GEMM_3XTF32
from oracle import ref

from _util import TOL, assert_gemm_close

pytestmark = pytest.mark.gpu
f32 = np.float32


def host_split_lo(x: np.ndarray) -> np.ndarray:
    """x minus x with its 13 low mantissa bits cleared (exact), plus half a tf32 unit on the magnitude so that a
    truncating reader rounds to nearest: the definition of the lo plane, restated on the host."""
    u = x.view(np.uint32)
    d = x - (u & np.uint32(0xFFFFE000)).view(f32)
    return (d.view(np.uint32) + np.uint32(0x1000)).view(f32)


def test_split_lo_matches_its_definition():
    for n in (1, 3, 4, 1000, 100003, 1 << 20):
        x = workloads.normal(n, n)
        got = linalg.split_lo(linalg.Tensor(x)).numpy()
        assert np.array_equal(got.view(np.uint32), host_split_lo(x).view(np.uint32)), n
    # hi + lo carries the value to 22 bits: |x - (trunc(x) + lo)| <= 2^-22 |x|
    x = workloads.uniform_pm1(9, 4096)
    lo = linalg.split_lo(linalg.Tensor(x)).numpy()
    hi = (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(f32)
    tf32_lo = (lo.view(np.uint32) & np.uint32(0xFFFFE000)).view(f32)
    assert np.max(np.abs(x.astype(np.float64) - hi - tf32_lo) / np.abs(x)) <= 2.0 ** -21


# (m, n, k, trans_a, trans_b, algo): lo-plane route, in-kernel split, padded planes on one CTA (ragged extents),
# CTA pairs, the exact kernel, the narrow transposed route's shape
ROUTES = [(1024, 1024, 512, False, False, GEMM_AUTO), (4096, 1024, 256, False, True, GEMM_AUTO),
          (512, 2048, 384, True, False, GEMM_AUTO), (300, 200, 100, False, False, GEMM_3XTF32),
          (4352, 4096, 160, False, False, GEMM_3XTF32), (96, 80, 40, False, False, GEMM_EXACT),
          (4096, 64, 2048, False, False, GEMM_3XTF32), (1024, 512, 2048, False, False, GEMM_AUTO)]   # last: split-K


@pytest.mark.parametrize("m,n,k,ta,tb,algo", ROUTES)
def test_output_lo_plane_equals_a_split_of_the_result_and_changes_nothing(m, n, k, ta, tb, algo):
    a, b = workloads.gemm_inputs(m, n, k)
    A = linalg.Tensor(np.ascontiguousarray(a.T) if ta else a)
    B = linalg.Tensor(np.ascontiguousarray(b.T) if tb else b)
    plain = linalg.gemm_into(linalg.Tensor.empty(m, n), A, B, trans_a=ta, trans_b=tb, algo=algo)
    c_lo = linalg.Tensor.filled(7.0, m, n)
    fused = linalg.gemm_into(linalg.Tensor.empty(m, n), A, B, trans_a=ta, trans_b=tb, algo=algo, c_lo=c_lo)
    cb.sync()
    if not (m == 4096 and n == 64):   # the narrow route is not taken with a lo output: same tolerance, other bits
        assert np.array_equal(fused.numpy(), plain.numpy())
    else:
        assert_gemm_close(fused.numpy(), a, b, what="narrow shape with a lo output")
    assert np.array_equal(c_lo.numpy().view(np.uint32), host_split_lo(fused.numpy()).view(np.uint32))


@pytest.mark.parametrize("m,n,k,ta,tb", [(1024, 1024, 512, False, False), (2048, 2048, 1024, True, False),
                                         (512, 4096, 256, False, True), (4096, 1024, 4096, True, False)])
def test_operand_lo_planes_from_the_caller_change_no_bit(m, n, k, ta, tb):
    a, b = workloads.gemm_inputs(m, n, k)
    A = linalg.Tensor(np.ascontiguousarray(a.T) if ta else a)
    B = linalg.Tensor(np.ascontiguousarray(b.T) if tb else b)
    bias = linalg.Tensor(workloads.uniform_pm1(5, n))
    A_lo, B_lo = linalg.split_lo(A), linalg.split_lo(B)
    L = cb.lib()
    plain = linalg.gemm_into(linalg.Tensor.empty(m, n), A, B, trans_a=ta, trans_b=tb, bias=bias, act="tanh")
    before = L.cleave_cuda_kernel_launches()
    fused = linalg.gemm_into(linalg.Tensor.empty(m, n), A, B, trans_a=ta, trans_b=tb, bias=bias, act="tanh",
                             a_lo=A_lo, b_lo=B_lo)
    assert L.cleave_cuda_kernel_launches() - before == 1          # no operand pre-pass
    half = linalg.gemm_into(linalg.Tensor.empty(m, n), A, B, trans_a=ta, trans_b=tb, bias=bias, act="tanh", b_lo=B_lo)
    cb.sync()
    assert np.array_equal(fused.numpy(), plain.numpy()) and np.array_equal(half.numpy(), plain.numpy())
    z = ref.bias_add(ref.matmul(a, b), bias.numpy())
    s = ref.matmul_absdot(a, b) + np.abs(bias.numpy())
    assert np.max(np.abs(fused.numpy().astype(np.float64) - ref.tanh(z)) / s) <= TOL


def test_mse_gradient_lo_plane():
    y = ref.sigmoid(workloads.normal(3, 512, 256))
    t = workloads.uniform01(4, 512, 256)
    Y, T = linalg.Tensor(y), linalg.Tensor(t)
    loss_dev = linalg.Tensor.zero(1)
    dz, dz_lo = nn.mse_act_bwd_lo(Y, T, "sigmoid", loss_dev)
    want_loss, want_dz = nn.mse_act_bwd(Y, T, "sigmoid")
    assert loss_dev[0] == want_loss and np.array_equal(dz.numpy(), want_dz.numpy())
    assert np.array_equal(dz_lo.numpy().view(np.uint32), host_split_lo(dz.numpy()).view(np.uint32))


@pytest.mark.parametrize("batch,d_in,d_hid,d_out", [(512, 256, 1024, 256), (1024, 512, 2048, 128)])
def test_chained_perceptron_step_is_bit_identical_to_the_unchained_one(batch, d_in, d_hid, d_out):
    X, W1, b1, W2, b2, T = workloads.mlp_inputs(batch, d_in, d_hid, d_out)
    b1 = workloads.uniform_pm1(41, d_hid) * f32(0.1)
    tX, tT = linalg.Tensor(X), linalg.Tensor(T)
    nets = [autodiff.MLP2(d_in, d_hid, d_out, chain_lo=flag) for flag in (False, True)]
    L = cb.lib()
    out, launches = [], []
    for net in nets:
        net.load(W1, b1, W2, b2)
        before = L.cleave_cuda_kernel_launches()
        loss = net.forward_backward(tX, tT)
        launches.append(L.cleave_cuda_kernel_launches() - before)
        cb.sync()
        out.append((loss, net.grads.numpy().copy()))
    assert out[0][0] == out[1][0]
    assert np.array_equal(out[0][1], out[1][1])
    # the chained step adds at most the three plane passes over X, W1 and W2 (the other planes leave epilogues)
    assert launches[1] <= launches[0] + 3, launches
    want = ref.mlp2_fwd_bwd(X, W1, b1, W2, b2, T)
    absX = np.abs(X).astype(np.float64)
    adZ1 = np.abs(want["dZ1"]).astype(np.float64)
    err = np.max(np.abs(nets[1].dW1.numpy().astype(np.float64) - want["dW1"]) / (absX.T @ adZ1))
    assert err <= TOL


@pytest.mark.parametrize("rows,d_in,d_out", [(64, 32, 48), (300, 100, 52), (4096, 1024, 1024), (2048, 4096, 1024)])
def test_dense_grads_equals_the_product_followed_by_the_column_sums(rows, d_in, d_out):
    # dw = x^T dz and db = colsum(dz) in one call, the sums queued beside the product on the library's second
    # stream: bit for bit the two-call form, with and without the operands' lo planes, and repeatedly (the fork and
    # join must leave the library's stream ordered: every round reads what the previous one wrote)
    T = linalg.Tensor
    x = workloads.uniform_pm1(rows + 1, rows, d_in)
    dz = workloads.normal(rows + 2, rows, d_out)
    tx, tdz = T(x), T(dz)
    want_dw = linalg.gemm_into(T.empty(d_in, d_out), tx, tdz, trans_a=True).numpy()
    want_db = nn.colsum(tdz).numpy()
    assert np.max(np.abs(want_db.astype(np.float64) - ref.colsum(dz)) / np.sum(np.abs(dz), axis=0)) <= TOL
    for planes in (False, True):
        x_lo = linalg.split_lo(tx) if planes else None
        dz_lo = linalg.split_lo(tdz) if planes else None
        for _ in range(3):
            dw, db = T.filled(7.0, d_in, d_out), T.filled(7.0, d_out)
            linalg.dense_grads(dw, db, tx, tdz, x_lo, dz_lo)
            got_db = db.numpy()
            assert np.array_equal(got_db, want_db)
            if planes:
                want_planes = linalg.gemm_into(T.empty(d_in, d_out), tx, tdz, trans_a=True, a_lo=x_lo, b_lo=dz_lo).numpy()
                assert np.array_equal(dw.numpy(), want_planes)
            else:
                assert np.array_equal(dw.numpy(), want_dw)
    with pytest.raises(Exception):
        linalg.dense_grads(T.empty(d_in, d_out), T.empty(d_out + 1), tx, tdz)
