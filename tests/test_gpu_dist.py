"""Data-parallel step on two GPUs (one process per GPU, NCCL) against the full-batch
CPU restatement.  Skipped on boxes with a single GPU; the arithmetic of the
exchange is also covered on CPU by test_dist_cpu.py."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

DIMS, GLOBAL_BATCH, STEPS, LR, SEED = [64, 96, 48, 10], 256, 3, 0.05, 5


def _worker(rank: int, world: int, conn_id, out_q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import rstorch_b200 as rt
    from rstorch_b200 import synth
    from test_gpu_train import build_mlp, linears
    ctx = rt.Context(rank)
    comm_id = conn_id.recv()
    comm = rt.Communicator(ctx, rank, world, comm_id)
    model = build_mlp(ctx, DIMS, synth.mlp_weights(SEED, DIMS), identity=False)
    loss_fn, opt = rt.CrossEntropyLoss(), rt.SGD.new(LR)
    first, rows = rt.shard_rows(GLOBAL_BATCH, rank, world)
    stats = []
    for s in range(STEPS):
        X, T = synth.gaussian_batch(SEED, s, first, rows, DIMS[0], DIMS[-1], GLOBAL_BATCH)
        x, t = ctx.tensor(X), ctx.tensor(T)
        loss = loss_fn.forward(model.forward(x), t)
        stats.append((loss, loss_fn.last_accuracy))
        rt.backward_with_exchange(model, loss_fn.backward(), comm, need_input_grad=False)
        opt.step(model)
    ctx.synchronize()
    ctx.check_device()
    out_q.put((rank, stats, [(l.weight.numpy(), l.bias.numpy(), l.grad_weight.numpy()) for l in linears(model)]))
    comm.close()
    ctx.close()


def test_two_gpu_step_equals_full_batch_step():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import multiprocessing as mp

    from conftest import REL_TOL, rel_err
    from oracle import oracle_c as oc
    from rstorch_b200 import Communicator, synth
    ctx = mp.get_context("spawn")
    world = 2
    out_q = ctx.Queue()
    pipes = [ctx.Pipe(duplex=False) for _ in range(world)]
    procs = [ctx.Process(target=_worker, args=(r, world, pipes[r][0], out_q)) for r in range(world)]
    for p in procs:
        p.start()
    comm_id = Communicator.new_id()
    for _, send in pipes:
        send.send(comm_id)
    results = {}
    for _ in range(world):
        rank, stats, params = out_q.get(timeout=300)
        results[rank] = (stats, params)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0

    weights = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(SEED, DIMS)]
    for s in range(STEPS):
        X, T = synth.gaussian_batch(SEED, s, 0, GLOBAL_BATCH, DIMS[0], DIMS[-1], GLOBAL_BATCH)
        losses, accs, grads = oc.mlp_train(DIMS, weights, X, T, GLOBAL_BATCH, 1, LR, skip_first_dx=True)
        mean_loss = np.mean([results[r][0][s][0] for r in range(world)])     # mean of per-rank means
        mean_acc = np.mean([results[r][0][s][1] for r in range(world)])
        assert abs(mean_loss - losses[0]) <= REL_TOL * abs(losses[0])
        assert mean_acc == pytest.approx(accs[0], abs=1e-12)
    for r in range(world):
        for (w, b, dw), (w_ref, b_ref), (dw_ref, _) in zip(results[r][1], weights, grads):
            assert rel_err(w, w_ref) < REL_TOL and rel_err(b, b_ref) < REL_TOL
            assert rel_err(dw, dw_ref) < REL_TOL
    # replicas stay bit-identical: every rank applied the same averaged gradient
    for a, b in zip(results[0][1], results[1][1]):
        for u, v in zip(a, b):
            assert np.array_equal(u, v)
