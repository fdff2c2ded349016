"""cleave_b200: host-side mirror of cleave's tensor operator surface over ``libcleave_cuda``,
a hand-written sm_100a (B200) implementation behind a C ABI.

    from cleave_b200 import linalg, nn
    a = linalg.Tensor([[1, 2, 3], [4, 5, 6]]); b = linalg.Tensor([[7, 8], [9, 10], [11, 12]])
    c = linalg.matmul(a, b); c[0, 0]  # 58.0

There is no CPU fallback: the shared library must be built (``python -m cleave_b200.build``)
and a CUDA device must be present for any compute call to succeed.
"""
from . import _lib, autodiff, dp, linalg, nn, workloads  # noqa: F401
from ._lib import CleaveCudaError, lib  # noqa: F401
from .linalg import Tensor, matmul  # noqa: F401

__all__ = ["linalg", "nn", "autodiff", "dp", "workloads", "Tensor", "matmul", "CleaveCudaError", "lib"]


def sync() -> None:
    """Wait for all queued device work; raises if a kernel reported a failure."""
    if lib().cleave_cuda_sync() != 0:
        _lib.raise_last_error("sync")
