import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_sessionstart(session):
    # Bring the two shared libraries up to date with their sources (no-ops when they are fresh):
    # the device library the tests exercise and the CPU oracle they check it against.
    try:
        from cleave_b200 import build
        build.build()
    except Exception as e:  # no nvcc on this machine: the prebuilt library is used if present
        print(f"note: libcleave_cuda not rebuilt ({e})", file=sys.stderr)
    from oracle import ref
    ref.build()
