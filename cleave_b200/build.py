"""Builds ``libcleave_cuda.so`` in-tree with nvcc for sm_100a.

The library is plain CUDA C++ behind a C ABI (``include/cleave_cuda.h``); it links the CUDA
runtime statically and reaches the driver's tensor-map encoder through
``cudaGetDriverEntryPoint``, so it loads on a machine without a GPU (every compute call then
fails with ``CLEAVE_CUDA_ERR_NO_DEVICE``).

Each ``csrc/*.cu`` is compiled to an object of its own (in parallel, only when it or a header
changed) under ``csrc/_obj/`` and the objects are linked into the shared library.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libcleave_cuda.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers() -> list[str]:
    return glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(os.path.dirname(HERE), "include", "cleave_cuda.h")]


def _newer(deps: list[str], target: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel for sm_100a into ``cleave_b200/libcleave_cuda.so``; returns its path."""
    srcs = sources()
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in srcs]
    hdrs = _headers()
    todo = [(s, o) for s, o in zip(srcs, objs) if force or _newer([s] + hdrs, o)]
    if not todo and not _newer(objs, LIB):
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libcleave_cuda cannot be built")
    os.makedirs(OBJ, exist_ok=True)

    def compile_one(pair):
        src, obj = pair
        cmd = [nvcc, *NVCC_FLAGS, "-c", "-o", obj, src]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), file=sys.stderr)
        subprocess.check_call(cmd)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
        list(pool.map(compile_one, todo))
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
