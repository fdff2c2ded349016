"""The cut last wave of the CTA-pair GEMM: when the tile count is not a multiple of the SM-pair count and the last wave
fills at most half of the pairs, each of its tiles is cut along K into runs that different pairs add up, and a second
kernel adds the runs in K order.  CLEAVE_CUDA_GEMM_STREAMK is read once per process, so each setting runs in a child."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode):
    # CLEAVE_CUDA_GEMM_PAIR=1: shapes whose operands cannot be read in place (ragged n, transposed ragged m) take the
    # padded-planes route, which runs on CTA pairs only above 4096^2 outputs unless told to
    env = dict(os.environ, CLEAVE_CUDA_GEMM_STREAMK=mode, CLEAVE_CUDA_GEMM_PAIR="1")
    r = subprocess.run([sys.executable, os.path.join(HERE, "streamk_worker.py")], env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    last = r.stdout.strip().splitlines()[-1].split()
    assert last[0] == "OK"
    return int(last[1]), int(last[2])


def test_cut_and_uncut_last_wave_both_match_the_oracle():
    cases_off, launches_off = _run("0")
    cases_on, launches_on = _run("1")
    assert cases_off == cases_on
    # every product but the last one has a cut region (one more launch each: the second pass)
    assert launches_on == launches_off + 11
