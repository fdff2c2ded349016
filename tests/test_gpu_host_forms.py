"""The host-array entry points (what a lowering hook calls for operations on native cleave tensors): arrays in
host memory in, the result array out, against the CPU oracle."""
import ctypes

import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import workloads
from cleave_b200._lib import c_f32p
from oracle import ref

from _util import assert_gemm_close

pytestmark = pytest.mark.gpu
f32 = np.float32
OP = dict(add=1, sub=2, mul=3, div=4, neg=5, exp=6, tanh=7, relu=8, sigmoid=9)


def _p(a):
    return a.ctypes.data_as(c_f32p)


def test_reference_matmul_known_answer_through_host_arrays():
    # cleave/tests/mlir_lower.rs:2077-2089: [[1,2,3],[4,5,6]] * [[7,8],[9,10],[11,12]] = [[58,64],[139,154]]
    L = cb.lib()
    a = np.array([[1, 2, 3], [4, 5, 6]], f32)
    b = np.array([[7, 8], [9, 10], [11, 12]], f32)
    c = np.zeros((2, 2), f32)
    assert L.cleave_cuda_host_gemm_f32(_p(a), a.size, _p(b), b.size, _p(c), c.size, 2, 2, 3) == 4
    assert c.tolist() == [[58.0, 64.0], [139.0, 154.0]]


@pytest.mark.parametrize("m,n,k", [(512, 512, 512), (100, 260, 77), (2048, 1024, 640)])
def test_host_gemm_pageable_arrays(m, n, k):
    L = cb.lib()
    a, b = workloads.gemm_inputs(m, n, k)
    c = np.empty((m, n), f32)
    assert L.cleave_cuda_host_gemm_f32(_p(a), a.size, _p(b), b.size, _p(c), c.size, m, n, k) == c.size
    assert_gemm_close(c, a, b, what=("host_gemm", m, n, k))


def test_host_gemm_pinned_arrays_is_pipelined_over_row_blocks():
    # 2^33 multiply-adds and pinned arrays: row blocks of A are uploaded while earlier blocks are multiplied and
    # downloaded.  m is not a multiple of the block height, so the last block is short.
    L = cb.lib()
    m, n, k = 4096 + 640, 2048, 1024
    a, b = workloads.gemm_inputs(m, n, k)
    pins = [L.cleave_cuda_host_alloc(4 * x) for x in (m * k, m * n)]
    assert all(pins)
    try:
        ha = np.ctypeslib.as_array(ctypes.cast(pins[0], c_f32p), shape=(m, k))
        hc = np.ctypeslib.as_array(ctypes.cast(pins[1], c_f32p), shape=(m, n))
        ha[:] = a
        hc[:] = -7.0
        before = L.cleave_cuda_kernel_launches()
        assert L.cleave_cuda_host_gemm_f32(_p(ha), a.size, _p(b), b.size, _p(hc), hc.size, m, n, k) == m * n
        assert L.cleave_cuda_kernel_launches() - before > 3          # several row blocks, not one product
        rows = np.concatenate([np.arange(0, m, 37), np.arange(m - 8, m)])
        assert_gemm_close(np.ascontiguousarray(hc[rows]), np.ascontiguousarray(a[rows]), b, what="pipelined host_gemm")
        lhs = a.astype(np.float64).sum(axis=0) @ b.astype(np.float64)
        scale = np.abs(a).astype(np.float64).sum(axis=0) @ np.abs(b).astype(np.float64)
        assert np.max(np.abs(lhs - hc.astype(np.float64).sum(axis=0)) / scale) <= 1e-5
    finally:
        for p in pins:
            L.cleave_cuda_host_free(p)


def test_host_elementwise_forms_match_the_oracle():
    L = cb.lib()
    x = workloads.normal(3, 100003)
    y = workloads.normal(4, 100003) + f32(3.0)
    out = np.empty_like(x)
    for name in ("add", "sub", "mul", "div"):
        assert L.cleave_cuda_host_binary_f32(OP[name], _p(x), x.size, _p(y), y.size, _p(out), out.size) == x.size
        assert np.array_equal(out, getattr(ref, name)(x, y)), name
    for name in ("neg", "relu"):
        assert L.cleave_cuda_host_unary_f32(OP[name], _p(x), x.size, _p(out), out.size) == x.size
        assert np.array_equal(out, getattr(ref, name)(x)), name
    for name in ("exp", "tanh", "sigmoid"):
        assert L.cleave_cuda_host_unary_f32(OP[name], _p(x), x.size, _p(out), out.size) == x.size
        assert np.allclose(out, getattr(ref, name)(x), rtol=1e-5, atol=0), name


def test_host_forms_reject_inconsistent_lengths():
    L = cb.lib()
    x = np.ones(8, f32)
    out = np.ones(4, f32)
    assert L.cleave_cuda_host_unary_f32(OP["neg"], _p(x), 8, _p(out), 4) == -3
    assert L.cleave_cuda_host_binary_f32(99, _p(x), 8, _p(x), 8, _p(x), 8) == -4
    assert L.cleave_cuda_host_gemm_f32(_p(x), 8, _p(x), 8, _p(out), 4, 2, 2, 3) == -3
    L.cleave_cuda_clear_error()
