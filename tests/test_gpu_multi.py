"""Two-rank run of the sharded paths on real GPUs (skipped when fewer than two are visible)."""
import os
import socket
import subprocess
import sys

import pytest

import cleave_b200 as cb

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_data_parallel_training_and_row_block_gemm_on_two_gpus():
    if cb.lib().cleave_cuda_device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_dp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "multi-gpu worker ok" in r.stdout
