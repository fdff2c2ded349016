"""Bounded device waits and their host-side reporting, exercised without faulting or hanging the GPU: a wait is
made to run out by a flag that nothing sets, with the limit shortened to 50 ms (see failure_worker.py)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_status_word_timeout_of_the_exchange_kernel_and_recovery():
    env = dict(os.environ, CLEAVE_CUDA_DP_WAIT_MS="50")
    r = subprocess.run([sys.executable, os.path.join(HERE, "failure_worker.py")], env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "failure worker ok" in r.stdout


def test_call_trace_prints_operation_shape_and_time():
    code = ("import numpy as np, cleave_b200 as cb\n"
            "from cleave_b200 import linalg, nn, workloads\n"
            "a, b = workloads.gemm_inputs(256, 512, 128)\n"
            "c = linalg.matmul(linalg.Tensor(a), linalg.Tensor(b))\n"
            "s = nn.sum(c.reshape(256 * 512)); t = nn.tanh(c); cb.sync()\n")
    env = dict(os.environ, CLEAVE_CUDA_TRACE="1", PYTHONPATH=os.path.dirname(HERE))
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-4000:]
    lines = [ln for ln in r.stderr.splitlines() if ln.startswith("cleave_cuda trace:")]
    text = "\n".join(lines)
    assert "gemm" in text and "m=256 n=512 k=128" in text and "sum" in text and "tanh" in text, r.stderr[-2000:]
    assert all(ln.rstrip().endswith("us") for ln in lines)


def test_debug_guard_bytes_stay_intact_over_a_mixed_workload():
    code = ("import numpy as np, cleave_b200 as cb\n"
            "from cleave_b200 import autodiff, linalg, nn, workloads\n"
            "X, W1, b1, W2, b2, T = workloads.mlp_inputs(300, 68, 132, 36)\n"
            "net = autodiff.MLP2(68, 132, 36); net.load(W1, b1, W2, b2)\n"
            "for _ in range(3): net.forward_backward(linalg.Tensor(X), linalg.Tensor(T)); net.sgd(0.1)\n"
            "a, b = workloads.gemm_inputs(1000, 260, 516)\n"
            "c = linalg.gemm_into(linalg.Tensor.empty(1000, 260), linalg.Tensor(a), linalg.Tensor(b), algo=linalg.GEMM_3XTF32)\n"
            "v = linalg.Tensor(workloads.normal(1, 100003)); s = nn.sum(v + v); del c, v, net\n"
            "cb.sync(); cb.lib().cleave_cuda_reset()\n"
            "print('guard failures', cb.lib().cleave_cuda_test_hook(3, 0))\n")
    env = dict(os.environ, CLEAVE_CUDA_DEBUG="1", PYTHONPATH=os.path.dirname(HERE))
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-4000:]
    assert "guard failures 0" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
