"""Sharding of the tensor path across the GPUs of one box: one process per GPU.

The reference has no distribution at all ("named as a goal but not designed", doc/hld.md:250);
what shards here is what the benchmark configurations partition naturally:

* batched GEMM by batch index and large GEMM by row blocks of A / C -- independent units, no
  collective in the data path (``batch_shard``, ``row_block``, ``row_block_matmul``);
* data-parallel training of the two-layer perceptron -- the one real exchange step: after the local
  backward pass the contiguous gradient buffer is summed over ranks with one NCCL all-reduce
  (``torch.distributed``, over NVLink / NVSwitch) and the 1/G of the mean is folded into the SGD pass.

``torch`` is used for process-group plumbing and as a zero-copy view of the library's device
memory; all arithmetic stays in libcleave_cuda kernels.
"""
from __future__ import annotations

import ctypes

import numpy as np


def shard(n: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of the ``n`` units owned by ``rank``: contiguous, sizes differ by at most one."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def batch_shard(batch: int, rank: int, world: int) -> range:
    """Batch indices of a batched GEMM owned by ``rank`` (b -> rank b mod G, so work stays even
    when the batch is not a multiple of the world size)."""
    return range(rank, batch, world)


def row_block(m: int, rank: int, world: int, tile: int = 128) -> tuple[int, int]:
    """Rows of A and C owned by ``rank`` for a row-block sharded GEMM; block edges fall on
    multiples of the GEMM tile height so no tile straddles two ranks."""
    tiles = (m + tile - 1) // tile
    lo, hi = shard(tiles, rank, world)
    return min(lo * tile, m), min(hi * tile, m)


class _CudaArrayView:
    """Exposes a libcleave_cuda buffer through ``__cuda_array_interface__`` (no copy)."""

    def __init__(self, ptr: int, shape: tuple[int, ...]):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": "<f4", "data": (ptr, False), "version": 2}


def as_torch(t, offset: int = 0, numel: int | None = None):
    """Zero-copy torch view of (a slice of) a device ``Tensor``; the Tensor must outlive the view."""
    import torch
    n = t.numel - offset if numel is None else numel
    view = torch.as_tensor(_CudaArrayView(t.data_ptr + 4 * offset, (n,)), device="cuda")
    view._cleave_owner = t
    return view


def use_torch_stream():
    """Creates a torch stream, makes it current and points the library at it, so library kernels,
    NCCL collectives and torch CUDA events are all ordered on one stream.  Returns the stream."""
    import torch

    from ._lib import lib
    s = torch.cuda.Stream()
    torch.cuda.set_stream(s)
    lib().cleave_cuda_set_stream(ctypes.c_void_p(s.cuda_stream))
    return s


class DataParallel:
    """Synchronous data-parallel SGD over a replica that keeps its gradients in one flat buffer.

    ``replica`` provides ``forward_backward(X, T, on_grads_ready=...) -> loss``, ``grad_buckets()``
    (list of flat torch views over its gradient buffer, in the order the backward pass completes
    them) and ``sgd(lr, gscale)``.  Every rank sees a different shard of the global batch; after
    ``step`` all replicas hold identical parameters.
    """

    def __init__(self, replica, group=None, overlap: bool = True):
        import torch.distributed as dist
        self.replica, self.group, self.overlap = replica, group, overlap
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._dist = dist
        self._buckets = replica.grad_buckets()

    def step(self, X, T, lr: float, loss_out=None):
        dist, pending = self._dist, []

        def on_ready(i: int) -> None:
            # bucket i is final: start summing it while the rest of the backward pass runs
            if self.world > 1 and self.overlap:
                pending.append(dist.all_reduce(self._buckets[i], op=dist.ReduceOp.SUM, group=self.group,
                                               async_op=True))

        loss = self.replica.forward_backward(X, T, on_grads_ready=on_ready, loss_out=loss_out)
        if self.world > 1 and not self.overlap:
            for b in self._buckets:
                dist.all_reduce(b, op=dist.ReduceOp.SUM, group=self.group)
        for w in pending:
            w.wait()     # orders the current stream after the collective; does not block the host
        # mean of the per-rank gradients: the 1/G is applied inside the SGD kernel
        self.replica.sgd(lr, 1.0 / self.world)
        return loss


class FusedDataParallel:
    """Data-parallel SGD where the gradient sum, the update and the replication of the new weights
    are ONE libcleave_cuda kernel over NVLink peer memory (``cleave_cuda_dp_sgd_allreduce_f32``)
    instead of an NCCL all-reduce followed by an SGD pass.

    Parameters and gradients live in torch symmetric memory (the plumbing that allocates the same
    buffer on every rank and exchanges the peer / multicast addresses); ``make_net(params, grads)``
    must build the replica on those flat buffers.  ``multimem=True`` sums in the NVSwitch when
    the fabric offers a multicast address; ``False`` uses plain peer loads in rank order.
    """

    def __init__(self, n_params: int, make_net, group=None, multimem: bool = True):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from .linalg import Tensor
        if n_params % 4:
            raise ValueError("the flat parameter vector must be a multiple of 4 elements (16-byte words)")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self._bufs, self._hdls = [], []
        for n, dt in ((n_params, torch.float32), (n_params, torch.float32), (64, torch.int32)):
            t = symm.empty(n, dtype=dt, device=dev)
            t.zero_()
            self._bufs.append(t)
        torch.cuda.synchronize()
        for t in self._bufs:
            self._hdls.append(symm.rendezvous(t, self.group))
        dist.barrier(self.group)
        p, g, f = self._hdls
        self.multimem = bool(multimem and p.has_multicast_support and p.multicast_ptr and g.multicast_ptr)
        arr = ctypes.c_void_p * self.world
        self._tables = [arr(*[int(h.buffer_ptrs[r]) for r in range(self.world)]) for h in (p, g, f)]
        self._mc = (ctypes.c_void_p(int(p.multicast_ptr)), ctypes.c_void_p(int(g.multicast_ptr))) if self.multimem \
            else (None, None)
        self.n_params = n_params
        self.params = Tensor.from_device_ptr(self._bufs[0].data_ptr(), n_params)
        self.grads = Tensor.from_device_ptr(self._bufs[1].data_ptr(), n_params)
        self.net = make_net(self.params, self.grads)
        # Buckets in the replica's numbering: 0 = [W2 | b2], 1 = [W1 | b1]; the backward pass completes bucket 1 first.
        o = [int(x) for x in self.net._offsets]
        self._buckets = [(o[2], o[4] - o[2]), (o[0], o[2] - o[0])]
        if any(off % 4 or n % 4 for off, n in self._buckets):
            self._buckets = [(0, n_params)]          # ragged layer sizes: exchange everything at the end
        # Each bucket has its own signal words (32 apart), epoch counter and completion event.  Exchanges run
        # on a side stream: layer 1's beside the rest of the backward pass, layer 2's beside the next step's
        # first forward product; the main stream waits for a layer's exchange only where it next reads that layer.
        self._flag_tables = [arr(*[int(f.buffer_ptrs[r]) + 128 * b for r in range(self.world)])
                             for b in range(len(self._buckets))]
        self._epochs = [1] * len(self._buckets)
        self._main = torch.cuda.current_stream()
        from ._lib import lib
        if (lib().cleave_cuda_get_stream() or 0) != self._main.cuda_stream:
            raise RuntimeError("the library must run on torch's current stream: call dp.use_torch_stream() first")
        self._side = torch.cuda.Stream()
        self._ready = [torch.cuda.Event() for _ in self._buckets]
        self._done = [torch.cuda.Event() for _ in self._buckets]
        self._in_flight = [False] * len(self._buckets)
        self._torch = torch
        # Lo planes of the weights (what the tensor-core products read beside W itself), refreshed on the side stream
        # right after the exchange that rewrote the layer: the split of W1 / W2 leaves the step's critical path.
        # _planes[b] belongs to bucket b's weight matrix; valid only after that bucket's first exchange.
        self._planes = None
        if len(self._buckets) == 2:
            self._planes = [Tensor.empty(*self.net.W2.dims), Tensor.empty(*self.net.W1.dims)]
        self._planes_version = [-1, -1]   # net.weights_version at the refresh; a load() or sgd() since makes a plane stale

    def _exchange(self, b: int, lr: float, stream) -> None:
        from ._lib import lib, raise_last_error
        off, n = self._buckets[b]
        rc = lib().cleave_cuda_dp_sgd_allreduce_f32(self._tables[0], self._tables[1], self._flag_tables[b], self._mc[0],
                                                    self._mc[1], off, n, self.rank, self.world, float(lr),
                                                    self._epochs[b], ctypes.c_void_p(stream.cuda_stream))
        if rc != 0:
            raise_last_error("dp_sgd_allreduce")
        self._epochs[b] += 2

    def _settle(self, b: int) -> None:
        """The main stream continues only after bucket b's exchange in flight, if any."""
        if self._in_flight[b]:
            self._main.wait_event(self._done[b])
            self._in_flight[b] = False

    def flush(self) -> None:
        """Orders the main stream after every exchange still in flight (call before reading the parameters,
        timing the end of a run, or switching streams)."""
        for b in range(len(self._buckets)):
            self._settle(b)

    def step(self, X, T, lr: float, loss_out=None):
        """``loss_out``: optional one-element device tensor; with it the step never waits for the GPU.
        When the step returns, the exchange of the last bucket(s) may still be running on the side stream; the
        next ``step`` (or ``flush``) orders itself after it."""
        split = len(self._buckets) == 2

        def before_layer(i: int) -> None:
            # layer i's weights are about to be read: the previous step's exchange of them must have landed
            if split:
                self._settle(2 - i)       # layer 1 -> bucket 1, layer 2 -> bucket 0
            elif i == 1:
                self._settle(0)

        def on_ready(b: int) -> None:
            if not split:
                if b == 0:                # everything is final
                    self._launch(0, lr)
                return
            self._launch(b, lr)

        planes = None
        self._refresh_planes = self._planes is not None and self.net.chains_planes(X.dims[0])
        if self._refresh_planes:
            v = self.net.weights_version
            planes = (self._planes[1] if self._planes_version[1] == v else None,
                      self._planes[0] if self._planes_version[0] == v else None)
        loss = self.net.forward_backward(X, T, on_grads_ready=on_ready, loss_out=loss_out, before_layer=before_layer,
                                         weight_planes=planes)
        return loss

    def _launch(self, b: int, lr: float) -> None:
        from ._lib import lib, raise_last_error
        self._ready[b].record(self._main)
        self._side.wait_event(self._ready[b])
        self._exchange(b, lr, self._side)
        if self._planes is not None and getattr(self, "_refresh_planes", False):
            w = self.net.W2 if b == 0 else self.net.W1
            if lib().cleave_cuda_split_lo_into_f32(self._planes[b]._h, w._h, ctypes.c_void_p(self._side.cuda_stream)) != 0:
                raise_last_error("split_lo_into")
            self._planes_version[b] = self.net.weights_version
        self._done[b].record(self._side)
        self._in_flight[b] = True


class MLP2Replica:
    """Adapter of ``autodiff.MLP2`` to the ``DataParallel`` interface."""

    def __init__(self, net):
        self.net = net
        o = [int(x) for x in net._offsets]
        # bucket 0 = [W2 | b2], bucket 1 = [W1 | b1]; the backward pass completes bucket 1 first
        self._buckets = [as_torch(net.grads, o[2], o[4] - o[2]), as_torch(net.grads, o[0], o[2] - o[0])]

    def grad_buckets(self):
        return self._buckets

    def forward_backward(self, X, T, on_grads_ready=None, loss_out=None):
        return self.net.forward_backward(X, T, on_grads_ready=on_grads_ready, loss_out=loss_out)

    def sgd(self, lr, gscale):
        self.net.sgd(lr, gscale)


def row_block_matmul(a_rows, b_full, group=None, src: int = 0):
    """C rows of this rank for a row-block sharded GEMM.  ``a_rows`` is this rank's [rows, k] block
    of A; ``b_full`` is a [k, n] device Tensor whose contents are valid on rank ``src`` and are
    replicated into every rank's own HBM first (an NCCL broadcast), so the GEMM only ever reads
    local memory."""
    import torch.distributed as dist

    from .linalg import matmul
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(as_torch(b_full), src=src, group=group)
    return matmul(a_rows, b_full)


def dp_batch_inputs(global_batch: int, rank: int, world: int, d_in: int, d_out: int, step: int = 0):
    """This rank's shard of a seeded global batch: every rank draws from the same generator
    stream and keeps its own contiguous rows, so the union over ranks is independent of G."""
    from . import workloads
    lo, hi = shard(global_batch, rank, world)
    X = workloads.normal(1000 + step, global_batch, d_in)[lo:hi]
    T = workloads.uniform01(2000 + step, global_batch, d_out)[lo:hi]
    return np.ascontiguousarray(X), np.ascontiguousarray(T)
