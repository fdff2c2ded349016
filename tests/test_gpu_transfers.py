"""Asynchronous transfers: results equal the synchronous path, ordering hazards are respected."""
import ctypes

import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import linalg
from cleave_b200._lib import c_f32p
from oracle import ref

pytestmark = pytest.mark.gpu
f32 = np.float32


def pinned(L, n):
    p = L.cleave_cuda_host_alloc(4 * n)
    assert p
    return p, np.ctypeslib.as_array(ctypes.cast(p, c_f32p), shape=(n,))


def test_pipelined_upload_compute_download_matches_oracle():
    L = cb.lib()
    m = n = k = 256
    steps = 6
    pa, ha = pinned(L, m * k)
    pb, hb = pinned(L, k * n)
    pcs = [pinned(L, m * n) for _ in range(2)]
    A = [linalg.Tensor.empty(m, k) for _ in range(2)]
    B = [linalg.Tensor.empty(k, n) for _ in range(2)]
    C = [linalg.Tensor.empty(m, n) for _ in range(2)]
    rng = np.random.default_rng(0)
    inputs = [(rng.uniform(-1, 1, (m, k)).astype(f32), rng.uniform(-1, 1, (k, n)).astype(f32)) for _ in range(steps)]
    results = []

    def up(i, step):
        # the pinned staging buffers are reused, so the previous copy out of them must be finished
        assert L.cleave_cuda_transfers_sync() == 0
        ha[:] = inputs[step][0].ravel()
        hb[:] = inputs[step][1].ravel()
        assert L.cleave_cuda_upload_async_f32(A[i]._h, ha.ctypes.data_as(c_f32p), ha.size) == 0
        assert L.cleave_cuda_upload_async_f32(B[i]._h, hb.ctypes.data_as(c_f32p), hb.size) == 0

    up(0, 0)
    for s in range(steps):
        cur = s & 1
        linalg.gemm_into(C[cur], A[cur], B[cur], algo=linalg.GEMM_EXACT)
        assert L.cleave_cuda_download_async_f32(C[cur]._h, pcs[cur][1].ctypes.data_as(c_f32p), m * n) == 0
        if s + 1 < steps:
            up(1 - cur, s + 1)          # syncs transfers first: the download above has landed
        else:
            assert L.cleave_cuda_transfers_sync() == 0
        results.append(pcs[cur][1].reshape(m, n).copy())
    for s in range(steps):
        assert np.array_equal(results[s], ref.matmul(*inputs[s])), s
    for p, _ in [(pa, ha), (pb, hb)] + pcs:
        L.cleave_cuda_host_free(p)


def test_upload_async_waits_for_earlier_readers_and_later_users_wait_for_it():
    L = cb.lib()
    n = 1 << 22
    p1, h1 = pinned(L, n)
    p2, h2 = pinned(L, n)
    h1[:] = 1.0
    h2[:] = 2.0
    t = linalg.Tensor.empty(n)
    assert L.cleave_cuda_upload_async_f32(t._h, h1.ctypes.data_as(c_f32p), n) == 0
    a = t + t                                   # must see 1.0 everywhere: waits for the first upload
    assert L.cleave_cuda_upload_async_f32(t._h, h2.ctypes.data_as(c_f32p), n) == 0   # must not overtake the add
    b = t + t                                   # must see 2.0 everywhere
    assert (a.numpy() == 2.0).all() and (b.numpy() == 4.0).all()
    assert L.cleave_cuda_transfers_sync() == 0
    L.cleave_cuda_host_free(p1)
    L.cleave_cuda_host_free(p2)
