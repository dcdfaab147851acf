"""Data-parallel steps (one process per GPU, NCCL) against the full-batch CPU
restatement.  The small-network test needs two GPUs; the deep-MLP test runs at every
world size the box offers (1 included), so a single-GPU box still checks the benchmark's
own layer widths.  The arithmetic of the exchange is also covered on CPU by
test_dist_cpu.py."""
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


def _launch(target, world, extra_args=(), timeout=900):
    """Runs `target(rank, world, pipe, queue, *extra_args)` in `world` processes that share
    one communicator id; returns {rank: payload}."""
    import multiprocessing as mp

    from rstorch_b200 import Communicator
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    pipes = [ctx.Pipe(duplex=False) for _ in range(world)]
    procs = [ctx.Process(target=target, args=(r, world, pipes[r][0], out_q) + tuple(extra_args)) for r in range(world)]
    for p in procs:
        p.start()
    comm_id = Communicator.new_id() if world > 1 else b""
    for _, send in pipes:
        send.send(comm_id)
    results = {}
    try:
        for _ in range(world):
            item = out_q.get(timeout=timeout)
            results[item[0]] = item[1:]
    finally:
        for p in procs:
            p.join(timeout=120)
    for p in procs:
        assert p.exitcode == 0
    return results


def test_two_gpu_step_equals_full_batch_step():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from conftest import REL_TOL, rel_err
    from oracle import oracle_c as oc
    from rstorch_b200 import synth
    world = 2
    results = _launch(_worker, world, timeout=300)

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


# ---- the deep MLP at its own widths, reduced global batch ----------------------------------
DEEP_DIMS = [4096] + [8192] * 9 + [1000]
DEEP_BATCH, DEEP_LR, DEEP_SEED = 512, 0.01, 0
KEPT_LAYERS = (0, 5, 9)          # weights of these layers are kept from the 1-rank run for the cross-G check


def _deep_worker(rank: int, world: int, conn_id, out_q, keep_dir: str):
    """One step of the deep MLP on this rank's rows.  Every rank reports the digests of its
    updated weights; rank 0 also runs the full-batch CPU restatement in-process and compares
    every gradient and every updated weight with it (the other replicas are covered by
    the digests), so no weight matrix has to travel between processes."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import rstorch_b200 as rt
    from conftest import rel_err
    from rstorch_b200 import synth
    from test_gpu_train import build_mlp, linears
    ctx = rt.Context(rank)
    comm_id = conn_id.recv()
    comm = rt.Communicator(ctx, rank, world, comm_id) if world > 1 else None
    weights = synth.mlp_weights(DEEP_SEED, DEEP_DIMS)
    model = build_mlp(ctx, DEEP_DIMS, weights, identity=False)
    for lin in linears(model):
        lin._host_weight = lin._host_bias = None
    if rank != 0:
        del weights
    loss_fn, opt = rt.CrossEntropyLoss(), rt.SGD.new(DEEP_LR)
    first, rows = rt.shard_rows(DEEP_BATCH, rank, world)
    X, T = synth.gaussian_batch(DEEP_SEED, 0, first, rows, DEEP_DIMS[0], DEEP_DIMS[-1], DEEP_BATCH)
    loss = loss_fn.forward(model.forward(ctx.tensor(X)), ctx.tensor(T))
    acc = loss_fn.last_accuracy
    rt.backward_with_exchange(model, loss_fn.backward(), comm, need_input_grad=False)
    opt.step(model)
    ctx.synchronize()
    ctx.check_device()
    report = {"loss": loss, "acc": acc, "digests": [p.parm.checksum() for p in model.parameters()]}
    if rank == 0:
        from oracle import oracle_c as oc
        Xg, Tg = synth.gaussian_batch(DEEP_SEED, 0, 0, DEEP_BATCH, DEEP_DIMS[0], DEEP_DIMS[-1], DEEP_BATCH)
        losses, accs, grads = oc.mlp_train(DEEP_DIMS, weights, Xg, Tg, DEEP_BATCH, 1, DEEP_LR, skip_first_dx=True)
        report["ref_loss"], report["ref_acc"] = float(losses[0]), float(accs[0])
        errs = []
        for l, lin in enumerate(linears(model)):
            w = lin.weight.numpy()
            errs.append((rel_err(lin.grad_weight.numpy(), grads[l][0]), rel_err(lin.grad_bias.numpy(), grads[l][1]),
                         rel_err(w, weights[l][0]), rel_err(lin.bias.numpy(), weights[l][1])))
            if l in KEPT_LAYERS:
                path = os.path.join(keep_dir, f"w{l}.npy")
                if world == 1:
                    np.save(path, w)
                elif os.path.exists(path):
                    report.setdefault("vs_one_rank", []).append(rel_err(w, np.load(path)))
        report["errs"] = errs
    out_q.put((rank, report))
    if comm is not None:
        comm.close()
    ctx.close()


def test_deep_mlp_true_widths_at_every_world_size(tmp_path):
    """4096 -> 8192 -> 8 x (8192 -> 8192) -> 1000 (the benchmark's network) at a global batch
    of 512 rows, one step, at G = 1, 2, 4, 8 ranks as far as the box has GPUs: rank 0's
    gradients and updated weights against the full-batch CPU restatement within 1e-9, all
    replicas bit-identical (digests of every parameter), the batch loss as the mean of the
    shard losses, and the G-rank weights against the 1-rank weights within 1e-9 (layers 0, 5
    and 9 are kept from the 1-rank run for that)."""
    import torch

    from conftest import REL_TOL
    sizes = [int(v) for v in os.environ.get("RSTORCH_TEST_WORLD_SIZES", "1,2,4,8").split(",")]
    sizes = [g for g in sizes if g <= torch.cuda.device_count()]
    assert sizes, "no world size fits this box"
    for world in sizes:
        results = _launch(_deep_worker, world, extra_args=(str(tmp_path),), timeout=1500)
        head = results[0][0]
        worst = max(max(e) for e in head["errs"])
        assert worst < REL_TOL, (world, head["errs"])
        mean_loss = float(np.mean([results[r][0]["loss"] for r in range(world)]))
        mean_acc = float(np.mean([results[r][0]["acc"] for r in range(world)]))
        assert abs(mean_loss - head["ref_loss"]) <= REL_TOL * abs(head["ref_loss"]), world
        assert mean_acc == pytest.approx(head["ref_acc"], abs=1e-12)
        for r in range(1, world):
            assert results[r][0]["digests"] == head["digests"], (world, r)
        if world > 1 and 1 in sizes:
            assert len(head["vs_one_rank"]) == len(KEPT_LAYERS) and max(head["vs_one_rank"]) < REL_TOL, world
        print(f"G={world}: worst relative error against the restatement {worst:.3e}; replicas identical; "
              f"against one rank {max(head.get('vs_one_rank', [0.0])):.3e}")
