"""Failure-detection scenarios on ONE GPU, none of which faults, traps or hangs it.

Started by test_gpu_failure_detection.py as a child process with CLEAVE_CUDA_DP_WAIT_MS=50 (the wait limit is
read once per process).  Scenarios:

  status   the host-side path: a status code planted in the mapped status word (what a kernel writes when a
           bounded wait runs out) turns into CLEAVE_CUDA_ERR_DEVICE_TIMEOUT at the next synchronisation, the
           word is cleared and the library keeps working.
  timeout  the data-parallel exchange kernel is launched as rank 0 of a world of 2 whose second rank never
           signals (both "ranks'" buffers are local): the entry barrier runs into its 50 ms limit, the kernel
           returns, the status is reported -- and no weight on either "rank" has changed.
  replay   the same kernel with the peer's signals written in advance by the host, once as rank 0 and once as
           rank 1 (two launches one after the other, neither waits for the other): together they must perform
           the whole averaged SGD update, checked against the CPU oracle.
Prints ``failure worker ok`` at the end.
"""
import ctypes
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import cleave_b200 as cb  # noqa: E402
from cleave_b200 import linalg, nn  # noqa: E402
from oracle import ref  # noqa: E402

f32 = np.float32
ERR_DEVICE_TIMEOUT = 7
HOOK_SET_DEVICE_STATUS = 1


def table(*tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr for t in tensors])


def exchange(L, params, grads, flags, n, rank, lr, epoch):
    return L.cleave_cuda_dp_sgd_allreduce_f32(table(*params), table(*grads), table(*flags), None, None, 0, n, rank,
                                              len(params), lr, epoch, None)


def main():
    L = cb.lib()
    assert L.cleave_cuda_init(0) == 0

    # ---- status: host-side translation of the status word
    x = linalg.Tensor(np.arange(1000, dtype=f32))
    assert L.cleave_cuda_test_hook(HOOK_SET_DEVICE_STATUS, 10) == 0
    assert L.cleave_cuda_sync() == ERR_DEVICE_TIMEOUT
    msg = L.cleave_cuda_last_error_message()
    assert b"bounded wait" in msg and b"code 10" in msg, msg
    L.cleave_cuda_clear_error()
    assert L.cleave_cuda_sync() == 0                       # reported once, then cleared
    assert nn.sum(x) == float(np.arange(1000, dtype=np.float64).sum())
    # a scalar-returning call that meets a planted code fails with NaN and the same error, then recovers
    assert L.cleave_cuda_test_hook(HOOK_SET_DEVICE_STATUS, 3) == 0
    assert np.isnan(L.cleave_cuda_sum_f32(x._h)) and L.cleave_cuda_last_error() == ERR_DEVICE_TIMEOUT
    L.cleave_cuda_clear_error()
    assert nn.max_of(x) == 999.0

    # ---- timeout: the second rank never arrives
    n = 1 << 16
    rng = np.random.default_rng(5)
    w0 = rng.standard_normal(n).astype(f32)
    g = [rng.standard_normal(n).astype(f32) for _ in range(2)]
    params = [linalg.Tensor(w0), linalg.Tensor(w0)]
    grads = [linalg.Tensor(g[0]), linalg.Tensor(g[1])]
    flags = [linalg.Tensor.zero(64), linalg.Tensor.zero(64)]
    cb.sync()
    t0 = time.perf_counter()
    assert exchange(L, params, grads, flags, n, 0, 0.25, 1) == 0      # the launch itself succeeds
    rc = L.cleave_cuda_sync()
    waited = time.perf_counter() - t0
    assert rc == ERR_DEVICE_TIMEOUT, rc
    msg = L.cleave_cuda_last_error_message()
    assert b"code 10" in msg, msg                                      # the entry barrier gave up
    L.cleave_cuda_clear_error()
    assert 0.03 <= waited <= 1.5, waited                               # the 50 ms limit, not the 2 s default
    assert np.array_equal(params[0].numpy(), w0) and np.array_equal(params[1].numpy(), w0), "weights were touched"
    assert L.cleave_cuda_sync() == 0

    # ---- replay: both ranks' halves of a healthy exchange, one launch after the other
    flags = [linalg.Tensor.zero(64), linalg.Tensor.zero(64)]
    epoch = 1
    for rank in (0, 1):
        peer = 1 - rank
        pre = np.zeros(64, np.uint32)
        pre[peer] = epoch + 1                        # "the peer has signalled entry and exit of this epoch"
        flags[rank] = linalg.Tensor(pre.view(f32))
        cb.sync()
        assert exchange(L, params, grads, flags, n, rank, 0.25, epoch) == 0
        assert L.cleave_cuda_sync() == 0, L.cleave_cuda_last_error_message()
    mean_g = ref.mul(ref.add(g[0], g[1]), np.full(n, 0.5, f32))     # sum in rank order, then * 1/world
    want = ref.sgd(w0, mean_g, 0.25)
    for p in params:
        assert np.array_equal(p.numpy(), want), "averaged SGD update differs from the oracle"
    print("failure worker ok")


if __name__ == "__main__":
    main()
