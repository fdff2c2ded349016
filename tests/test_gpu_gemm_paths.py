"""The three operand paths of the tensor-core GEMM -- padded hi/lo planes, split inside the kernel,
lo planes beside the caller's own tensors -- against the oracle on the same problems.  The library chooses between them by shape; here each
is forced for a whole process (the switch is read once), so the worker runs as a child."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("mode,pair,pair_bk,lo_pair", [("0", "0", "32", "0"), ("2", "0", "32", "0"), ("3", "0", "32", "0"),
                                                        ("0", "1", "32", "0"), ("0", "1", "16", "0"), ("3", "0", "32", "1")])
def test_forced_operand_path(mode, pair, pair_bk, lo_pair):
    # pair = "1": the padded-planes path runs its 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2), with a
    # K-block of 32 or 16; lo_pair = "1": so does the lo-plane path, reading the caller's tensors in place
    # CLEAVE_CUDA_GEMM_STREAMK=0: the cut of a partly filled last wave adds a launch to some of these products; it has
    # its own test (test_gpu_streamk.py), here the launch counts are about the operand routes
    env = dict(os.environ, CLEAVE_CUDA_GEMM_DIRECT=mode, CLEAVE_CUDA_GEMM_PAIR=pair, CLEAVE_CUDA_GEMM_PAIR_BK=pair_bk,
               CLEAVE_CUDA_GEMM_LO_PAIR=lo_pair, CLEAVE_CUDA_GEMM_STREAMK="0")
    r = subprocess.run([sys.executable, os.path.join(HERE, "gemm_paths_worker.py")], env=env, capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    last = r.stdout.strip().splitlines()[-1].split()
    assert last[0] == "OK"
    gemms, unaddressable, launches, lo_eligible = int(last[2]), int(last[3]), int(last[4]), int(last[5])
    # the padded-planes path (0) launches two split kernels and the GEMM; the lo-plane path (3) one kernel that
    # writes both planes and the GEMM, falling back to the padded planes where it cannot read the operands in
    # place; the direct path (2) only the GEMM, except for operands that TMA cannot address
    want = {"0": 3 * gemms, "2": gemms + 2 * unaddressable, "3": 2 * lo_eligible + 3 * (gemms - lo_eligible)}[mode]
    assert launches == want


def test_the_short_k_pair_kernel_gives_the_bits_of_the_general_one():
    # K <= 256 without an epilogue runs on the pair kernel's variant with 16 drain warps; CLEAVE_CUDA_GEMM_SHORTK=0
    # keeps the general kernel.  Same problems, both ways round: every result byte must agree.
    digests = []
    for shortk in ("1", "0"):
        env = dict(os.environ, CLEAVE_CUDA_GEMM_DIRECT="0", CLEAVE_CUDA_GEMM_PAIR="1", CLEAVE_CUDA_GEMM_SHORTK=shortk)
        r = subprocess.run([sys.executable, os.path.join(HERE, "gemm_paths_worker.py")], env=env, capture_output=True,
                           text=True, timeout=900)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
        last = r.stdout.strip().splitlines()[-1].split()
        assert last[0] == "OK"
        digests.append(last[6])
    assert digests[0] == digests[1]
