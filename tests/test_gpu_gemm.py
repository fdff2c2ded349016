"""Parity of the MatMul family with the CPU oracle: the exact CUDA-core path bit for bit, the
tcgen05 3xTF32 path within 1e-5 (componentwise against sum|a||b|, and normwise)."""
import json
import os

import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import linalg, workloads
from cleave_b200.linalg import GEMM_3XTF32, GEMM_EXACT
from oracle import ref

from _util import TOL, assert_gemm_close, rel_err

pytestmark = pytest.mark.gpu
f32 = np.float32


def gemm(a, b, algo, trans_a=False, trans_b=False, bias=None, act="identity", batch=None):
    ta, tb = linalg.Tensor(a), linalg.Tensor(b)
    if batch is None:
        m = a.shape[1] if trans_a else a.shape[0]
        n = b.shape[0] if trans_b else b.shape[1]
        c = linalg.Tensor.empty(m, n)
    else:
        c = linalg.Tensor.empty(batch, a.shape[1], b.shape[2])
    linalg.gemm_into(c, ta, tb, trans_a=trans_a, trans_b=trans_b, algo=algo,
                     bias=linalg.Tensor(bias) if bias is not None else None, act=act)
    cb.sync()
    return c.numpy()


def test_reference_known_answers_exact():
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")) as f:
        kats = json.load(f)
    for case in kats["matmul"]:
        c = linalg.matmul(linalg.Tensor(case["a"]), linalg.Tensor(case["b"]))
        assert np.array_equal(c.numpy(), np.array(case["c"], f32)), case["cite"]
    c = linalg.matmul(linalg.Tensor([[1, 2, 3], [4, 5, 6]]), linalg.Tensor([[7, 8], [9, 10], [11, 12]]))
    assert (c[0, 0], c[0, 1], c[1, 0], c[1, 1]) == (58.0, 64.0, 139.0, 154.0)
    z = linalg.matmul(linalg.Tensor([[1, 2], [3, 4]]), linalg.Tensor.zero(2, 2))
    assert not z.numpy().any()


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (2, 2, 3), (7, 5, 3), (33, 65, 17), (64, 64, 16), (100, 130, 77),
                                   (128, 256, 64), (512, 512, 512)])
def test_exact_path_is_bit_identical_to_the_reference_loop(m, n, k):
    a, b = workloads.gemm_inputs(m, n, k)
    assert np.array_equal(gemm(a, b, GEMM_EXACT), ref.matmul(a, b))


def test_exact_path_transposed_and_batched():
    a, b = workloads.gemm_inputs(70, 50, 90)
    want = ref.matmul(a, b)
    assert np.array_equal(gemm(np.ascontiguousarray(a.T), b, GEMM_EXACT, trans_a=True), want)
    assert np.array_equal(gemm(a, np.ascontiguousarray(b.T), GEMM_EXACT, trans_b=True), want)
    A = workloads.uniform_pm1(11, 3, 20, 30)
    B = workloads.uniform_pm1(12, 3, 30, 10)
    got = gemm(A, B, GEMM_EXACT, batch=3)
    for i in range(3):
        assert np.array_equal(got[i], ref.matmul(A[i], B[i]))


# Shapes for the tensor-core path: one tile, one K-block; ragged in every dimension; several
# tiles per CTA; more tiles than SMs; K not a multiple of the K-block; tall / wide.
TC_SHAPES = [(128, 256, 16), (128, 256, 32), (128, 256, 64), (128, 256, 512), (256, 512, 128),
             (100, 200, 50), (129, 257, 33), (1, 1, 1), (5, 300, 7), (300, 5, 1000),
             (512, 512, 512), (1024, 1024, 1024), (2048, 4096, 256), (640, 768, 2048),
             # few tiles with a long K, and more tiles than SMs with a ragged last wave
             (128, 256, 4096), (256, 512, 2048), (384, 256, 1280), (128, 256, 8192), (4096, 1024, 1024),
             (2560, 2048, 768), (1920, 2560, 512)]


@pytest.mark.parametrize("m,n,k", TC_SHAPES)
def test_3xtf32_path_within_tolerance(m, n, k):
    a, b = workloads.gemm_inputs(m, n, k)
    got = gemm(a, b, GEMM_3XTF32)
    assert_gemm_close(got, a, b, what=(m, n, k))


def test_3xtf32_matches_exact_path_on_exactly_representable_data():
    # Small integers: every product and partial sum is exact in tf32 x tf32 -> f32.
    rng = np.random.default_rng(0)
    a = rng.integers(-8, 9, (256, 384)).astype(f32)
    b = rng.integers(-8, 9, (384, 512)).astype(f32)
    assert np.array_equal(gemm(a, b, GEMM_3XTF32), ref.matmul(a, b))


def test_3xtf32_identity_and_layout():
    # A = I picks out rows of B: any descriptor / swizzle / tile-decoding mistake shows as a permutation.
    n = 512
    b = workloads.uniform_pm1(5, n, n)
    got = gemm(np.eye(n, dtype=f32), b, GEMM_3XTF32)
    assert rel_err(got, b) <= 2e-6 and np.array_equal(np.argmax(got, axis=1), np.argmax(b, axis=1))
    a = workloads.uniform_pm1(6, n, n)
    got = gemm(a, np.eye(n, dtype=f32), GEMM_3XTF32)
    assert rel_err(got, a) <= 2e-6


@pytest.mark.parametrize("m,n,k", [(256, 512, 384), (130, 70, 200)])
def test_3xtf32_transposed_operands(m, n, k):
    a, b = workloads.gemm_inputs(m, n, k)
    want = ref.matmul(a, b)
    assert_gemm_close(gemm(np.ascontiguousarray(a.T), b, GEMM_3XTF32, trans_a=True), a, b, want, "tn")
    assert_gemm_close(gemm(a, np.ascontiguousarray(b.T), GEMM_3XTF32, trans_b=True), a, b, want, "nt")


def test_3xtf32_batched():
    A = workloads.uniform_pm1(21, 5, 256, 128)
    B = workloads.uniform_pm1(22, 5, 128, 512)
    got = gemm(A, B, GEMM_3XTF32, batch=5)
    for i in range(5):
        assert_gemm_close(got[i], A[i], B[i], what=f"batch {i}")


@pytest.mark.parametrize("act", ["identity", "tanh", "sigmoid", "relu"])
def test_3xtf32_fused_bias_activation(act):
    a, b = workloads.gemm_inputs(256, 512, 256)
    a *= f32(0.1)
    bias = workloads.uniform_pm1(7, 512)
    z = ref.bias_add(ref.matmul(a, b), bias)
    want = z if act == "identity" else getattr(ref, act)(z)
    got = gemm(a, b, GEMM_3XTF32, bias=bias, act=act)
    # activations are 1-Lipschitz here; compare on the scale of the pre-activation error bound
    s = ref.matmul_absdot(a, b) + np.abs(bias)
    assert np.max(np.abs(got.astype(np.float64) - want) / np.maximum(s, 1e-30)) <= TOL


def test_cleave_matmul_dispatch_at_512_cubed():
    # Benchmark configuration 0: C = A B, M = N = K = 512, uniform[-1,1).
    a, b = workloads.gemm_inputs(512, 512, 512)
    got = linalg.matmul(linalg.Tensor(a), linalg.Tensor(b)).numpy()
    e = assert_gemm_close(got, a, b, what="512^3 auto")
    print("512^3 errors:", e)


def test_large_gemm_sampled_rows():
    # 4096^3 is too slow for a full oracle pass in a test; check 64 sampled rows exactly as the
    # reference loop computes them, plus a checksum-of-rows identity on the whole result.
    m = n = k = 4096
    a, b = workloads.gemm_inputs(m, n, k)
    got = gemm(a, b, GEMM_3XTF32)
    rows = np.random.default_rng(0).choice(m, 64, replace=False)
    a_s = np.ascontiguousarray(a[rows])
    assert_gemm_close(np.ascontiguousarray(got[rows]), a_s, b, what="4096^3 sampled rows")
    # linearity: (1^T A) B == 1^T (A B)
    lhs = (a.astype(np.float64).sum(axis=0) @ b.astype(np.float64))
    rhs = got.astype(np.float64).sum(axis=0)
    scale = np.abs(a).astype(np.float64).sum(axis=0) @ np.abs(b).astype(np.float64)
    assert np.max(np.abs(lhs - rhs) / scale) <= TOL


def test_non_finite_and_extreme_operands():
    # NaN propagates on both paths; the exact path follows the reference for infinities;
    # values next to FLT_MAX must not overflow in the hi/lo split.
    a, b = workloads.gemm_inputs(128, 256, 64)
    a[3, 5] = np.nan
    got = gemm(a, b, GEMM_3XTF32)
    want = ref.matmul(a, b)
    assert np.isnan(got[3]).all() and np.isnan(want[3]).all()
    ok = np.ones(128, bool)
    ok[3] = False
    assert_gemm_close(np.ascontiguousarray(got[ok]), np.ascontiguousarray(a[ok]), b, what="rows without NaN")
    a[3, 5] = np.inf
    with np.errstate(all="ignore"):
        assert np.array_equal(gemm(a, b, GEMM_EXACT), ref.matmul(a, b), equal_nan=True)
    big = np.zeros((128, 32), f32)
    big[:, 0] = np.float32(3.4028234e38)          # FLT_MAX: rounds to infinity in tf32 unless truncated
    one = np.zeros((32, 256), f32)
    one[0, :] = 0.5
    got = gemm(big, one, GEMM_3XTF32)
    assert np.isfinite(got).all() and np.allclose(got, np.float32(3.4028234e38) * 0.5, rtol=1e-6)


@pytest.mark.parametrize("algo", [GEMM_EXACT, GEMM_3XTF32])
@pytest.mark.parametrize("act", ["tanh", "sigmoid", "relu"])
def test_backward_form_equals_product_then_derivative(algo, act):
    # C = act'(y) * (A B): the fused epilogue must give, bit for bit, what the product followed by the
    # elementwise derivative kernel gives, and the oracle's composition within the GEMM tolerance.
    from cleave_b200 import nn
    for (m, n, k, ta, tb) in [(256, 512, 128, False, True), (130, 72, 200, False, False), (4096, 1024, 256, False, True),
                              (200, 260, 64, True, False)]:
        a, b = workloads.gemm_inputs(m, n, k)
        y = getattr(ref, act)(workloads.uniform_pm1(33, m, n))          # a plausible forward output
        A = linalg.Tensor(np.ascontiguousarray(a.T) if ta else a)
        B = linalg.Tensor(np.ascontiguousarray(b.T) if tb else b)
        Y = linalg.Tensor(y)
        fused = linalg.gemm_into(linalg.Tensor.empty(m, n), A, B, trans_a=ta, trans_b=tb, algo=algo, dact_of=Y, dact=act)
        prod = linalg.gemm_into(linalg.Tensor.empty(m, n), A, B, trans_a=ta, trans_b=tb, algo=algo)
        two_step = getattr(nn, act + "_bwd")(Y, prod)
        cb.sync()
        assert np.array_equal(fused.numpy(), two_step.numpy()), (m, n, k, act)
        want = getattr(ref, act + "_bwd")(y, ref.matmul(a, b))
        s = ref.matmul_absdot(a, b)
        assert np.max(np.abs(fused.numpy().astype(np.float64) - want) / np.maximum(s, 1e-30)) <= TOL


def test_backward_form_rejects_bad_arguments():
    a, b = workloads.gemm_inputs(64, 64, 64)
    A, B = linalg.Tensor(a), linalg.Tensor(b)
    with pytest.raises(TypeError):
        linalg.gemm_into(linalg.Tensor.empty(64, 64), A, B, dact_of=linalg.Tensor.empty(64, 32), dact="tanh")
    with pytest.raises(TypeError):
        linalg.gemm_into(linalg.Tensor.empty(64, 64), A, B, bias=linalg.Tensor(np.zeros(64, f32)),
                         dact_of=linalg.Tensor.empty(64, 64), dact="tanh")
    c = linalg.Tensor.empty(64, 64)
    L = cb.lib()
    r = L.cleave_cuda_gemm_dact_f32(c._h, A._h, B._h, 1, 64, 64, 64, 0, 0, 0, c._h, 3)
    assert r < 0 and b"alias" in (L.cleave_cuda_last_error_message() or b"")
    L.cleave_cuda_clear_error()


def test_seeded_random_shapes_through_every_dispatch_decision():
    # 40 seeded problems with arbitrary (also odd) extents, layouts and algorithms: whatever route the
    # library picks -- exact, in-kernel split, lo planes, padded planes -- the result obeys the same bound.
    rng = np.random.default_rng(20260)
    for case in range(40):
        m, n, k = (int(rng.integers(1, 700)) for _ in range(3))
        if case % 4 == 0:            # force TMA-addressable extents now and then
            m, n, k = (max(4, x // 4 * 4) for x in (m, n, k))
        ta, tb = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        algo = [linalg.GEMM_AUTO, GEMM_3XTF32, GEMM_EXACT][int(rng.integers(0, 3))]
        a = workloads.uniform_pm1(1000 + case, m, k)
        b = workloads.uniform_pm1(2000 + case, k, n)
        got = gemm(np.ascontiguousarray(a.T) if ta else a, np.ascontiguousarray(b.T) if tb else b, algo,
                   trans_a=ta, trans_b=tb)
        want = ref.matmul(a, b)
        if algo == GEMM_EXACT:
            assert np.array_equal(got, want), (case, m, n, k, ta, tb)
        else:
            assert_gemm_close(got, a, b, want, (case, m, n, k, ta, tb, algo))


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True)])
def test_pair_kernel_route_sampled_rows(trans_a, trans_b):
    # Outputs above 4096^2 take the padded-planes route on CTA pairs (256 x 256 tiles, tcgen05 cta_group::2).
    # 96 sampled rows are checked as the reference loop computes them, plus the linearity checksum over
    # the whole result; m is not a multiple of 256 so the last tile-row is ragged.
    m, n, k = 8192 + 136, 4096, 1536
    a, b = workloads.gemm_inputs(m, n, k)
    got = gemm(np.ascontiguousarray(a.T) if trans_a else a, np.ascontiguousarray(b.T) if trans_b else b,
               GEMM_3XTF32, trans_a=trans_a, trans_b=trans_b)
    rows = np.concatenate([np.random.default_rng(1).choice(m, 88, replace=False), np.arange(m - 8, m)])
    assert_gemm_close(np.ascontiguousarray(got[rows]), np.ascontiguousarray(a[rows]), b, what=("pair", trans_a, trans_b))
    lhs = a.astype(np.float64).sum(axis=0) @ b.astype(np.float64)
    rhs = got.astype(np.float64).sum(axis=0)
    scale = np.abs(a).astype(np.float64).sum(axis=0) @ np.abs(b).astype(np.float64)
    assert np.max(np.abs(lhs - rhs) / scale) <= TOL


@pytest.mark.parametrize("m,n,k", [(4096, 64, 4096), (2048, 40, 2048), (8192, 8, 2048), (2304, 64, 6144), (4096, 128, 4096),
                                   (2048, 100, 2560)])
def test_narrow_output_takes_the_transposed_split_k_route(m, n, k):
    # n <= 128 with long m and k: C^T = B^T A^T with K cut into slices, then one sum-and-transpose pass.
    a, b = workloads.gemm_inputs(m, n, k)
    L = cb.lib()
    before = L.cleave_cuda_kernel_launches()
    got = gemm(a, b, GEMM_3XTF32)
    assert L.cleave_cuda_kernel_launches() - before == 2          # the GEMM kernel and the sum-transpose pass
    assert_gemm_close(got, a, b, what=("narrow", m, n, k))


@pytest.mark.parametrize("m,n,k,ta,tb", [(1024, 1024, 1024, False, False), (512, 768, 4096, False, False),
                                         (1024, 512, 2048, True, False), (640, 1024, 1536, False, True),
                                         (256, 256, 8192, True, True), (1000, 520, 2048, False, False)])
def test_few_tiles_take_the_split_k_route(m, n, k, ta, tb):
    # Fewer tiles than half the SMs: K is cut into slices that run side by side, then one pass adds the partial
    # results in slice order and applies bias + activation.  Same tolerance as every other route.
    a, b = workloads.gemm_inputs(m, n, k)
    a *= f32(0.25)
    A = np.ascontiguousarray(a.T) if ta else a
    B = np.ascontiguousarray(b.T) if tb else b
    L = cb.lib()
    before = L.cleave_cuda_kernel_launches()
    got = gemm(A, B, linalg.GEMM_AUTO, trans_a=ta, trans_b=tb)
    assert L.cleave_cuda_kernel_launches() - before == 2          # the sliced GEMM kernel and the slice-sum pass
    assert_gemm_close(got, a, b, what=("split-K", m, n, k, ta, tb))
    bias = workloads.uniform_pm1(7, n)
    got = gemm(A, B, linalg.GEMM_AUTO, trans_a=ta, trans_b=tb, bias=bias, act="tanh")
    z = ref.bias_add(ref.matmul(a, b), bias)
    s = ref.matmul_absdot(a, b) + np.abs(bias)
    assert np.max(np.abs(got.astype(np.float64) - ref.tanh(z)) / s) <= TOL
    # run to run the same bits (fixed slice order)
    assert np.array_equal(got, gemm(A, B, linalg.GEMM_AUTO, trans_a=ta, trans_b=tb, bias=bias, act="tanh"))
