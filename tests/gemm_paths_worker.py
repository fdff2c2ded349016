"""Runs the tensor-core GEMM over a fixed list of problems and checks each against the CPU oracle.

Started by test_gpu_gemm_paths.py with CLEAVE_CUDA_GEMM_DIRECT set, because the library reads that
switch once per process: 0 sends every problem through the padded-planes pre-pass, 2 makes the kernel
split every operand that TMA can address, 3 uses the lo-plane pre-pass wherever it applies.  Prints one line
``OK <cases> <gemm calls> <calls TMA cannot address> <kernel launches> <calls the lo-plane route can serve>
<sha256 of every result's bytes>`` on success.
"""
import hashlib
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

# (m, n, k): one tile; ragged edges with 4-element alignment (direct path) and without (pre-pass only);
# row counts that are / are not multiples of 32 (blocked / plain MN-major boxes); narrow C; long K.
SHAPES = [(128, 256, 16), (128, 256, 64), (256, 512, 128), (100, 200, 52), (132, 260, 36), (4, 4, 4),
          (8, 300, 8), (300, 8, 1000), (512, 512, 512), (1024, 1024, 1024), (640, 768, 2048),
          (128, 256, 8192), (2560, 2048, 768), (4096, 64, 2048), (2048, 40, 512), (136, 72, 264),
          (129, 257, 33), (5, 300, 7)]


DIGEST = hashlib.sha256()
CALLS = {"gemms": 0, "unaddressable": 0, "other": 0, "lo_eligible": 0}


def run(a, b, trans_a=False, trans_b=False, bias=None, act="identity", batch=None):
    CALLS["gemms"] += 1
    # TMA needs every operand's contiguous extent to be a multiple of 4 elements (16 bytes)
    CALLS["unaddressable"] += int(a.shape[-1] % 4 != 0 or b.shape[-1] % 4 != 0)
    # the lo-plane route also needs whole 32-wide blocks of an operand that is read row-index-contiguous
    mm = a.shape[-1] if trans_a else a.shape[-2]
    nn_ = b.shape[-2] if trans_b else b.shape[-1]
    CALLS["lo_eligible"] += int(a.shape[-1] % 4 == 0 and b.shape[-1] % 4 == 0 and (not trans_a or mm % 32 == 0)
                                and (trans_b or nn_ % 32 == 0))
    ta, tb = linalg.Tensor(a), linalg.Tensor(b)
    if batch is None:
        m = a.shape[1] if trans_a else a.shape[0]
        n = b.shape[0] if trans_b else b.shape[1]
        c = linalg.Tensor.empty(m, n)
    else:
        c = linalg.Tensor.empty(batch, a.shape[1], b.shape[2])
    linalg.gemm_into(c, ta, tb, trans_a=trans_a, trans_b=trans_b, algo=GEMM_3XTF32,
                     bias=linalg.Tensor(bias) if bias is not None else None, act=act)
    cb.sync()
    out = c.numpy()
    DIGEST.update(out.tobytes())
    return out


def main() -> int:
    cases = 0
    for (m, n, k) in SHAPES:
        a, b = workloads.gemm_inputs(m, n, k)
        want = ref.matmul(a, b)
        assert_gemm_close(run(a, b), a, b, want, ("nn", m, n, k))
        assert_gemm_close(run(np.ascontiguousarray(a.T), b, trans_a=True), a, b, want, ("tn", m, n, k))
        assert_gemm_close(run(a, np.ascontiguousarray(b.T), trans_b=True), a, b, want, ("nt", m, n, k))
        assert_gemm_close(run(np.ascontiguousarray(a.T), np.ascontiguousarray(b.T), trans_a=True, trans_b=True),
                          a, b, want, ("tt", m, n, k))
        cases += 4
    # batched, with a ragged tile in every batch entry
    A = workloads.uniform_pm1(21, 3, 200, 96)
    B = workloads.uniform_pm1(22, 3, 96, 264)
    got = run(A, B, batch=3)
    for i in range(3):
        assert_gemm_close(got[i], A[i], B[i], what=("batch", i))
    cases += 1
    # fused epilogue
    a, b = workloads.gemm_inputs(256, 512, 256)
    a *= f32(0.1)
    bias = workloads.uniform_pm1(7, 512)
    z = ref.bias_add(ref.matmul(a, b), bias)
    s = ref.matmul_absdot(a, b) + np.abs(bias)
    for act in ("identity", "tanh", "sigmoid", "relu"):
        want = z if act == "identity" else getattr(ref, act)(z)
        got = run(a, b, bias=bias, act=act)
        assert np.max(np.abs(got.astype(np.float64) - want) / np.maximum(s, 1e-30)) <= TOL, act
        cases += 1
    # backward form: act'(y) * (a b) in the epilogue equals the product followed by the derivative kernel
    from cleave_b200 import nn
    y = ref.tanh(workloads.uniform_pm1(33, 256, 512))
    ta_, tb_, ty_ = linalg.Tensor(a), linalg.Tensor(b), linalg.Tensor(y)
    fused = linalg.gemm_into(linalg.Tensor.empty(256, 512), ta_, tb_, algo=GEMM_3XTF32, dact_of=ty_, dact="tanh")
    prod = linalg.gemm_into(linalg.Tensor.empty(256, 512), ta_, tb_, algo=GEMM_3XTF32)
    CALLS["gemms"] += 2
    CALLS["lo_eligible"] += 2
    before = cb.lib().cleave_cuda_kernel_launches()
    two_step = nn.tanh_bwd(ty_, prod)
    CALLS["other"] = cb.lib().cleave_cuda_kernel_launches() - before      # not a GEMM launch
    cb.sync()
    assert np.array_equal(fused.numpy(), two_step.numpy())
    cases += 1
    # exactly representable data: both paths must reproduce the reference loop bit for bit
    rng = np.random.default_rng(0)
    a = rng.integers(-8, 9, (256, 384)).astype(f32)
    b = rng.integers(-8, 9, (384, 512)).astype(f32)
    assert np.array_equal(run(a, b), ref.matmul(a, b))
    # values next to FLT_MAX stay finite; a NaN stays in its row
    big = np.zeros((128, 32), f32)
    big[:, 0] = f32(3.4028234e38)
    one = np.zeros((32, 256), f32)
    one[0, :] = 0.5
    got = run(big, one)
    assert np.isfinite(got).all() and np.allclose(got, f32(3.4028234e38) * 0.5, rtol=1e-6)
    a, b = workloads.gemm_inputs(128, 256, 64)
    a[3, 5] = np.nan
    got = run(a, b)
    assert np.isnan(got[3]).all() and not np.isnan(np.delete(got, 3, axis=0)).any()
    cases += 3
    print("OK", cases, CALLS["gemms"], CALLS["unaddressable"], cb.lib().cleave_cuda_kernel_launches() - CALLS["other"],
          CALLS["lo_eligible"], DIGEST.hexdigest())
    return 0


if __name__ == "__main__":
    sys.exit(main())
