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

__all__ = ["linalg", "nn", "autodiff", "dp", "workloads", "Tensor", "matmul", "CleaveCudaError", "lib", "StepGraph", "sync"]


def sync() -> None:
    """Wait for all queued device work; raises if a kernel reported a failure."""
    if lib().cleave_cuda_sync() != 0:
        _lib.raise_last_error("sync")


class StepGraph:
    """A step captured once into a CUDA graph and replayed (``cleave_cuda_graph_begin / _end / _launch / _free``).

        step = lambda: net.forward_backward(X, T, loss_out=loss)   # only calls that do not wait
        g = StepGraph(step)          # runs the step once (one-time kernel set-up), then captures it
        for _ in range(n): g.replay()

    Tensors the step allocates come from a cache that belongs to the graph, so the replays keep using exactly those
    blocks and nothing else is handed them; a tensor that outlives the step (an output) is overwritten by every replay.
    """

    def __init__(self, step, warm: bool = True):
        L = lib()
        if warm:
            step()
        if L.cleave_cuda_graph_begin() != 0:
            _lib.raise_last_error("graph_begin")
        try:
            self.result = step()
        finally:
            self._h = L.cleave_cuda_graph_end()
        if not self._h:
            _lib.raise_last_error("graph_end")

    def replay(self) -> None:
        if lib().cleave_cuda_graph_launch(self._h) != 0:
            _lib.raise_last_error("graph_launch")

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().cleave_cuda_graph_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:   # noqa: BLE001 - interpreter shutdown
            pass
