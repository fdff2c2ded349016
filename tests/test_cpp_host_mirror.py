"""The C++ host mirror (include/cleave_cuda.hpp) over the C ABI: the reference's known-answer tests
written the way the reference writes them, as a C++ program.  Without a GPU it must compile, link
against the library and refuse to compute; on a GPU it must reproduce every answer."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    from cleave_b200 import build
    lib = build.build()
    exe = str(tmp_path / "host_mirror_kats")
    gxx = shutil.which("g++")
    assert gxx, "g++ not found"
    cmd = [gxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "host_mirror_kats.cpp"), "-o", exe,
           "-L", os.path.dirname(lib), "-lcleave_cuda", f"-Wl,-rpath,{os.path.dirname(lib)}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def test_cpp_mirror_builds_and_has_no_cpu_fallback(tmp_path):
    exe = _build(tmp_path)
    from cleave_b200 import lib
    if lib().cleave_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "no CPU fallback" in r.stdout


@pytest.mark.gpu
def test_cpp_mirror_reproduces_the_reference_answers(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout[-2000:] + r.stderr[-2000:]
