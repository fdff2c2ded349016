"""Products whose last wave of 256 x 256 tiles is partly filled, through the CTA-pair kernel with and without the
cut of that wave along K (the library reads CLEAVE_CUDA_GEMM_STREAMK once per process), each against the CPU oracle.

Started by test_gpu_streamk.py.  Prints ``OK <cases> <kernel launches>`` on success.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import cleave_b200 as cb  # noqa: E402
from cleave_b200 import linalg, workloads  # noqa: E402
from cleave_b200.linalg import GEMM_3XTF32  # noqa: E402
from oracle import ref  # noqa: E402

from _util import TOL, assert_gemm_close  # noqa: E402

f32 = np.float32
T = linalg.Tensor


def main() -> int:
    cases = 0
    before = cb.lib().cleave_cuda_kernel_launches()
    # 10 x 8 = 80 tiles on 74 SM pairs, K = 2048 (64 K-blocks): the 6 tiles of the second wave are cut into 8 runs each;
    # ragged last tile-row and -column
    m, n, k = 2500, 2040, 2048
    a, b = workloads.gemm_inputs(m, n, k)
    want = ref.matmul(a, b)
    got = linalg.gemm_into(T.empty(m, n), T(a), T(b), algo=GEMM_3XTF32).numpy()
    assert_gemm_close(got, a, b, want, ("nn", m, n, k))
    at, bt = np.ascontiguousarray(a.T), np.ascontiguousarray(b.T)
    got = linalg.gemm_into(T.empty(m, n), T(at), T(b), trans_a=True, algo=GEMM_3XTF32).numpy()
    assert_gemm_close(got, a, b, want, ("tn", m, n, k))
    got = linalg.gemm_into(T.empty(m, n), T(a), T(bt), trans_b=True, algo=GEMM_3XTF32).numpy()
    assert_gemm_close(got, a, b, want, ("nt", m, n, k))
    cases += 3
    # bias + tanh in the second pass as in the tile epilogue, and the lo plane of the result
    a2 = a * f32(0.05)
    bias = workloads.uniform_pm1(7, n)
    z = ref.bias_add(ref.matmul(a2, b), bias)
    s = ref.matmul_absdot(a2, b) + np.abs(bias)
    for act in ("tanh", "sigmoid", "relu"):
        c, c_lo = T.empty(m, n), T.empty(m, n)
        linalg.gemm_into(c, T(a2), T(b), algo=GEMM_3XTF32, bias=T(bias), act=act, c_lo=c_lo)
        got = c.numpy()
        want_act = getattr(ref, act)(z)
        assert np.max(np.abs(got.astype(np.float64) - want_act) / np.maximum(s, 1e-30)) <= TOL, act
        assert np.array_equal(c_lo.numpy(), linalg.split_lo(c).numpy()), act   # the plane a consumer would compute itself
        cases += 1
    # backward form: tanh'(y) * (a b)
    y = ref.tanh(workloads.uniform_pm1(33, m, n))
    got = linalg.gemm_into(T.empty(m, n), T(a2), T(b), algo=GEMM_3XTF32, dact_of=T(y), dact="tanh").numpy()
    want_d = ref.tanh_bwd(y, ref.matmul(a2, b))
    assert np.max(np.abs(got.astype(np.float64) - want_d) / np.maximum(ref.matmul_absdot(a2, b), 1e-30)) <= TOL
    cases += 1
    # two batch entries of 10 x 8 tiles each (160 tiles, 12 of them cut into 6 runs): the cut tiles all belong to the
    # second entry
    A = workloads.uniform_pm1(21, 2, 2560, 2048)
    B = workloads.uniform_pm1(22, 2, 2048, 2048)
    got = linalg.gemm_into(T.empty(2, 2560, 2048), T(A), T(B), algo=GEMM_3XTF32).numpy()
    for i in range(2):
        assert_gemm_close(got[i], A[i], B[i], what=("batch", i))
    cases += 1
    # exactly representable data: the sum of K-runs reproduces the reference loop bit for bit
    rng = np.random.default_rng(0)
    ai = rng.integers(-8, 9, (2560, 2048)).astype(f32)
    bi = rng.integers(-8, 9, (2048, 2048)).astype(f32)
    got = linalg.gemm_into(T.empty(2560, 2048), T(ai), T(bi), algo=GEMM_3XTF32).numpy()
    assert np.array_equal(got, ref.matmul(ai, bi))
    cases += 1
    # K = 1024 (32 K-blocks): the 6 tiles of the second wave are cut into 4 runs of 8 K-blocks
    m, n, k = 2560, 2048, 1024
    a, b = workloads.gemm_inputs(m, n, k)
    got = linalg.gemm_into(T.empty(m, n), T(a), T(b), algo=GEMM_3XTF32).numpy()
    assert_gemm_close(got, a, b, what=("short runs", m, n, k))
    cases += 1
    # K = 768 (24 K-blocks, three runs of 8), both operands stored the other way round
    m, n, k = 2560, 2048, 768
    a, b = workloads.gemm_inputs(m, n, k)
    got = linalg.gemm_into(T.empty(m, n), T(np.ascontiguousarray(a.T)), T(np.ascontiguousarray(b.T)), trans_a=True,
                           trans_b=True, algo=GEMM_3XTF32).numpy()
    assert_gemm_close(got, a, b, what=("tt", m, n, k))
    cases += 1
    # fewer tiles than SM pairs (8 x 8 = 64): a single, nearly full wave is never cut
    m, n, k = 2048, 2048, 4096
    a, b = workloads.gemm_inputs(m, n, k)
    got = linalg.gemm_into(T.empty(m, n), T(a), T(b), algo=GEMM_3XTF32).numpy()
    rows = np.arange(0, m, 37)
    a_s = np.ascontiguousarray(a[rows])
    assert_gemm_close(np.ascontiguousarray(got[rows]), a_s, b, what=("64 tiles", m, n, k))
    cases += 1
    cb.sync()
    print("OK", cases, cb.lib().cleave_cuda_kernel_launches() - before)
    return 0


if __name__ == "__main__":
    sys.exit(main())
