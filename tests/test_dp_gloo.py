"""Host logic of the multi-GPU paths, run as world-size-2 gloo ranks on CPU.

The device library cannot run here, so the replica is a CPU stand-in built on the oracle
(tests may use the oracle; the product never does).  What is under test is the host side:
sharding of units, gradient buckets, the all-reduce + 1/G scaling, and that two ranks end with
identical parameters equal to single-process training on the whole batch.
"""
import os
import socket

import numpy as np
import pytest

from cleave_b200 import dp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_covers_every_unit_once():
    for n in (1, 7, 64, 100, 16384):
        for world in (1, 2, 3, 4, 8):
            spans = [dp.shard(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        dp.shard(10, 2, 2)


def test_batch_shard_and_row_blocks():
    for world in (1, 2, 4, 8):
        owned = sorted(b for r in range(world) for b in dp.batch_shard(64, r, world))
        assert owned == list(range(64))
        assert all(len(dp.batch_shard(64, r, world)) == 64 // world for r in range(world))
        blocks = [dp.row_block(16384, r, world) for r in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == 16384
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
        assert all(lo % 128 == 0 for lo, _ in blocks)
    assert dp.row_block(130, 0, 2) == (0, 128) and dp.row_block(130, 1, 2) == (128, 130)


class OracleReplica:
    """CPU stand-in with the interface DataParallel expects; arithmetic by the oracle."""

    def __init__(self, W1, b1, W2, b2):
        import torch
        from oracle import ref
        self.ref, self.torch = ref, torch
        self.shapes = [W1.shape, b1.shape, W2.shape, b2.shape]
        self.sizes = [int(np.prod(s)) for s in self.shapes]
        self.params = np.concatenate([a.ravel() for a in (W1, b1, W2, b2)]).astype(np.float32)
        self.grads = torch.zeros(self.params.size, dtype=torch.float32)
        o = np.concatenate([[0], np.cumsum(self.sizes)])
        self.o = o
        self._buckets = [self.grads[o[2]:o[4]], self.grads[o[0]:o[2]]]

    def _p(self):
        return [self.params[self.o[i]:self.o[i + 1]].reshape(self.shapes[i]) for i in range(4)]

    def grad_buckets(self):
        return self._buckets

    def forward_backward(self, X, T, on_grads_ready=None, loss_out=None):
        W1, b1, W2, b2 = self._p()
        r = self.ref.mlp2_fwd_bwd(X, W1, b1, W2, b2, T)
        g = np.concatenate([r[k].ravel() for k in ("dW1", "db1", "dW2", "db2")])
        self.grads.copy_(self.torch.from_numpy(g))
        if on_grads_ready:
            on_grads_ready(0)
            on_grads_ready(1)
        return float(r["loss"])

    def sgd(self, lr, gscale):
        self.params = self.ref.sgd(self.params, self.grads.numpy() * np.float32(gscale), lr)


def _worker(rank, world, port, overlap, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cleave_b200 import workloads
    _, W1, b1, W2, b2, _ = workloads.mlp_inputs(8, 12, 20, 6)
    rep = OracleReplica(W1, b1, W2, b2)
    trainer = dp.DataParallel(rep, overlap=overlap)
    losses = []
    for step in range(5):
        X, T = dp.dp_batch_inputs(16, rank, world, 12, 6, step)
        losses.append(trainer.step(X, T, 0.5))
    np.save(os.path.join(out, f"params_{rank}.npy"), rep.params)
    np.save(os.path.join(out, f"losses_{rank}.npy"), np.array(losses))
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("overlap", [False, True])
def test_two_gloo_ranks_match_single_process_training(tmp_path, overlap):
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, overlap, str(tmp_path)), nprocs=world, join=True)
    p0, p1 = (np.load(tmp_path / f"params_{r}.npy") for r in range(2))
    assert np.array_equal(p0, p1)            # replicas stay bit-identical
    # single process on the whole global batch: the mean over equal shards of per-shard mean
    # gradients is the full-batch mean gradient (up to float32 rounding of the two-step mean)
    from cleave_b200 import workloads
    from oracle import ref
    _, W1, b1, W2, b2, _ = workloads.mlp_inputs(8, 12, 20, 6)
    rep = OracleReplica(W1, b1, W2, b2)
    for step in range(5):
        X, T = dp.dp_batch_inputs(16, 0, 1, 12, 6, step)
        rep.forward_backward(X, T)
        rep.sgd(0.5, 1.0)
    assert np.allclose(p0, rep.params, rtol=1e-5, atol=1e-6)
    l0, l1 = (np.load(tmp_path / f"losses_{r}.npy") for r in range(2))
    assert l0.shape == l1.shape == (5,) and not np.array_equal(l0, l1)   # different shards


def test_dp_batch_inputs_union_is_independent_of_world_size():
    whole_X, whole_T = dp.dp_batch_inputs(32, 0, 1, 8, 4, step=3)
    for world in (2, 4):
        parts = [dp.dp_batch_inputs(32, r, world, 8, 4, step=3) for r in range(world)]
        assert np.array_equal(np.concatenate([p[0] for p in parts]), whole_X)
        assert np.array_equal(np.concatenate([p[1] for p in parts]), whole_T)
