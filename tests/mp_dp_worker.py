"""Worker of the multi-GPU test: run under torchrun with 2+ ranks, one GPU each.

Trains a small MLP data-parallel for a few steps through the device library + NCCL, checks that
the replicas stay identical and that the result matches oracle training on the whole batch.
Exits non-zero on any mismatch.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def train_and_check(torch, dist, cb, autodiff, dp, linalg, workloads, ref, rank, world, d_in, d_hid, d_out, gb, steps, lr):
    _, W1, b1, W2, b2, _ = workloads.mlp_inputs(1, d_in, d_hid, d_out)
    n_params = d_in * d_hid + d_hid + d_hid * d_out + d_out
    for overlap in ("nccl", "nccl-overlap", "fused-p2p", "fused-multimem"):
        if overlap.startswith("nccl"):
            net = autodiff.MLP2(d_in, d_hid, d_out)
            trainer = dp.DataParallel(dp.MLP2Replica(net), overlap=overlap.endswith("overlap"))
        else:
            trainer = dp.FusedDataParallel(
                n_params, lambda p, g: autodiff.MLP2(d_in, d_hid, d_out, params=p, grads=g),
                multimem=overlap.endswith("multimem"))
            net = trainer.net
            if rank == 0:
                print(f"{overlap}: multimem in use = {trainer.multimem}", flush=True)
        net.load(W1, b1, W2, b2)
        dist.barrier()
        for step in range(steps):
            X, T = dp.dp_batch_inputs(gb, rank, world, d_in, d_out, step)
            trainer.step(linalg.Tensor(X), linalg.Tensor(T), lr)
        if hasattr(trainer, "flush"):
            trainer.flush()          # the last exchanges run on a side stream
        cb.sync()
        mine = dp.as_torch(net.params).clone()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        for g in gathered[1:]:
            assert torch.equal(g, gathered[0]), "replicas diverged"
        # oracle: single-process training on the whole global batch
        P = [W1.copy(), b1.copy(), W2.copy(), b2.copy()]
        for step in range(steps):
            X, T = dp.dp_batch_inputs(gb, 0, 1, d_in, d_out, step)
            r = ref.mlp2_fwd_bwd(X, *P, T)
            P = [ref.sgd(p, r[k], lr) for p, k in zip(P, ("dW1", "db1", "dW2", "db2"))]
        want = np.concatenate([p.ravel() for p in P])
        got = mine.cpu().numpy()
        err = np.max(np.abs(got - want)) / np.max(np.abs(want))
        assert err <= 1e-5, f"mode={overlap}: parameters differ from whole-batch training by {err}"
        if rank == 0:
            print(f"{overlap}: ok, max deviation from whole-batch training {err:.2e}", flush=True)


def main():
    import torch
    import torch.distributed as dist

    import cleave_b200 as cb
    from cleave_b200 import autodiff, dp, linalg, workloads
    from oracle import ref

    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert cb.lib().cleave_cuda_init(local) == 0
    dp.use_torch_stream()
    # a small network (exact GEMM path) and one large enough for the tensor-core path with lo planes handed from
    # product to product and the weights' planes refreshed on the exchange stream
    for (d_in, d_hid, d_out, gb, steps, lr) in ((64, 256, 32, 512, 6, 0.5), (256, 512, 128, 512 * world, 5, 0.5)):
        train_and_check(torch, dist, cb, autodiff, dp, linalg, workloads, ref, rank, world, d_in, d_hid, d_out, gb, steps, lr)
    # row-block sharded GEMM with B broadcast into local HBM
    m, n, k = 1024, 512, 256
    a, b = workloads.gemm_inputs(m, n, k)
    lo, hi = dp.row_block(m, rank, world)
    tb = linalg.Tensor(b if rank == 0 else np.zeros_like(b))
    c = dp.row_block_matmul(linalg.Tensor(np.ascontiguousarray(a[lo:hi])), tb).numpy()
    want = ref.matmul_rows(a, b, lo, hi - lo)
    s = ref.matmul_absdot(np.ascontiguousarray(a[lo:hi]), b)
    assert np.max(np.abs(c - want) / s) <= 1e-5
    dist.barrier()
    if rank == 0:
        print("multi-gpu worker ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
