"""World-size-2 check of the data-parallel arithmetic on CPU (gloo): each rank
runs the restated step on its shard, gradients are averaged across ranks, and the
result must equal the full-batch step.  This is the host logic of the multi-GPU
path (sharding + averaging); the device side replaces gloo by NCCL."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    from oracle import oracle_c as oc
    from rstorch_b200 import shard_rows, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        oc.set_threads(1)
        dims, B, lr = [24, 16, 6], 32, 0.01
        weights = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(1, dims)]
        first, rows = shard_rows(B, rank, world)
        X, T = synth.gaussian_batch(1, 0, first, rows, dims[0], dims[-1], B)
        # local step with lr = 0 leaves the weights alone and yields the local gradients
        losses, accs, grads = oc.mlp_train(dims, weights, X, T, rows, 1, 0.0)
        flat = torch.from_numpy(np.concatenate([g.ravel() for pair in grads for g in pair]))
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
        flat /= world                                     # average of per-rank means
        stats = torch.tensor([losses[0], accs[0]])
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        stats /= world
        # apply SGD with the averaged gradients
        o = 0
        new = []
        for (w, b), (dw, db) in zip(weights, grads):
            gw = flat[o:o + dw.size].numpy().reshape(dw.shape); o += dw.size
            gb = flat[o:o + db.size].numpy().reshape(db.shape); o += db.size
            new.append((oc.sgd_step(w, gw, lr), oc.sgd_step(b, gb, lr)))
        if rank == 0:
            q.put((stats.numpy(), [(w, b) for w, b in new]))
    finally:
        dist.destroy_process_group()


def test_two_rank_average_equals_full_batch_step():
    sys.path.insert(0, ROOT)
    from conftest import REL_TOL, rel_err
    from oracle import oracle_c as oc
    from rstorch_b200 import synth
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    stats, new = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    dims, B, lr = [24, 16, 6], 32, 0.01
    weights = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(1, dims)]
    X, T = synth.gaussian_batch(1, 0, 0, B, dims[0], dims[-1], B)
    losses, accs, _ = oc.mlp_train(dims, weights, X, T, B, 1, lr)
    assert abs(stats[0] - losses[0]) <= REL_TOL * abs(losses[0])
    assert stats[1] == pytest.approx(accs[0], abs=1e-15)
    for (w, b), (wr, br) in zip(weights, new):
        assert rel_err(wr, w) < REL_TOL and rel_err(br, b) < REL_TOL
