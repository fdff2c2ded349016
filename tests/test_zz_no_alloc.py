"""The allocation-free sum entry point, called through the C ABI with raw device pointers.

It exists for callers that cannot allocate device memory at the point where they need the
reduction (another framework owns the heap, a cudaMalloc stall is unacceptable, the process is
at its memory budget).  Its result must equal the pooled entry point's, call after call: the
scratch array is shared by every call and keeps the previous call's contents, so the second call
here uses different data and a different length to show that nothing stale leaks through.
This file sorts last on purpose, so a run that stops at the first failure has already run
everything else.
"""
import ctypes

import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import linalg, nn
from oracle import ref

pytestmark = pytest.mark.gpu


def _sum_noalloc(L, t: linalg.Tensor, out: linalg.Tensor) -> float:
    stream = L.cleave_cuda_get_stream()          # queue behind the library's own work
    rc = L.cleave_cuda_sum_noalloc_f32(ctypes.c_void_p(t.data_ptr), t.numel, ctypes.c_void_p(out.data_ptr),
                                       ctypes.c_void_p(stream))
    assert rc == 0, L.cleave_cuda_last_error_message()
    return out[0]


def test_sum_noalloc_matches_the_pooled_sum_on_two_calls_in_a_row():
    L = cb.lib()
    rng = np.random.default_rng(7)
    first = linalg.Tensor(rng.standard_normal(3_000_001).astype(np.float32))
    second = linalg.Tensor((rng.standard_normal(70_001) * 100).astype(np.float32))
    out = linalg.Tensor.zero(1)
    want_first, want_second = nn.sum(first), nn.sum(second)
    live_before = L.cleave_cuda_live_bytes()
    got_first = _sum_noalloc(L, first, out)
    got_second = _sum_noalloc(L, second, out)
    assert L.cleave_cuda_live_bytes() == live_before          # no handle, no pool block taken
    # against the CPU oracle's f64 sum, on the scale of the sum of |terms|
    x1, x2 = first.numpy(), second.numpy()
    assert abs(got_first - ref.sum_f64(x1)) <= 1e-5 * ref.sum_abs_f64(x1)
    assert abs(got_second - ref.sum_f64(x2)) <= 1e-5 * ref.sum_abs_f64(x2)
    # and against the pooled entry point: same tree, same bits
    assert got_first == want_first and got_second == want_second


def test_sum_noalloc_recovers_from_a_stale_completion_word():
    # A call whose kernel was cut short would leave a partial count in the completion counter behind the partials.
    # Such values are planted here from the host (the test hook copies 8 bytes into the array; it launches
    # nothing).  Every following call must still write its output, and the right one.
    L = cb.lib()
    rng = np.random.default_rng(11)
    data = rng.standard_normal(5_000_000).astype(np.float32)
    t = linalg.Tensor(data)
    want = nn.sum(t)
    assert abs(want - ref.sum_f64(data)) <= 1e-5 * ref.sum_abs_f64(data)
    warm = linalg.Tensor.zero(1)
    assert _sum_noalloc(L, t, warm) == want                   # first call on this device looks the array up
    for stale in ((0x7FFF0000 << 32) | 5, -1, 37):
        cb.sync()
        assert L.cleave_cuda_test_hook(2, stale) == 0         # CLEAVE_HOOK_POISON_NOALLOC_WORD
        out = linalg.Tensor.filled(-1.0, 1)
        assert _sum_noalloc(L, t, out) == want
        assert _sum_noalloc(L, t, out) == want                # and the call after it


def test_sum_noalloc_rejects_sizes_it_cannot_handle():
    L = cb.lib()
    t = linalg.Tensor(np.ones(8, np.float32))
    out = linalg.Tensor.zero(1)
    p, o = ctypes.c_void_p(t.data_ptr), ctypes.c_void_p(out.data_ptr)
    assert L.cleave_cuda_sum_noalloc_f32(p, 1 << 31, o, None) == -8      # beyond the maximum
    assert b"exceed the maximum" in L.cleave_cuda_last_error_message()
    assert L.cleave_cuda_sum_noalloc_f32(p, 0, o, None) == -4
    assert L.cleave_cuda_sum_noalloc_f32(None, 8, o, None) == -4
    L.cleave_cuda_clear_error()
    assert _sum_noalloc(L, t, out) == 8.0                                # still usable afterwards
