#!/usr/bin/env python
"""Benchmark of the f64 training step (forward + loss + backward [+ all-reduce] + SGD).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5]
                    [--impl ours|reference]

Prints ONE JSON line.  The default workload is the deep MLP that the headline
metric is quoted on at 1/2/4/8 GPUs: 4096 -> 8192 -> 8 x (8192 -> 8192) -> 1000
(10 Linear layers, ReLU between them), f64, global batch 65536 split evenly over
the ranks (strong scaling), SGD lr 0.01, gradients averaged with NCCL before the
single-launch SGD step.  Inputs are seeded synthetic data of that shape.

`value` times the step with the batch already in HBM; `e2e` times the same step
fed from pinned host memory through the staging ring (host-to-device copy of the
batch and device-to-host read of loss/accuracy inside the timed region).
`--impl reference` times the CPU restatement of the reference's step on the host
cores (the reference itself is Rust over un-vendored crates and cannot be built
with the toolchains of this image).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (layer widths, global batch, input stream, leading Identity)
    "c1": ([784, 100, 100, 10], 32, "mnist_like", True),
    "c2": ([784, 100, 100, 10], 4096, "mnist_like", True),
    "c3": ([1024, 4096, 4096, 4096, 1000], 8192, "gaussian", False),
    "c4": ([4096] + [8192] * 9 + [1000], 65536, "gaussian", False),
}
WORKLOAD_NAMES = {
    "c1": "README MLP 784-100-100-10, batch 32",
    "c2": "MLP 784-100-100-10, batch 4096",
    "c3": "wide MLP 1024-4096-4096-4096-1000, batch 8192",
    "c4": "deep MLP 4096-8192-8x(8192-8192)-1000 (10 Linear), global batch 65536",
    "c5": "fused SGD step over 2^30 f64 parameters in 64 tensors",
}
LR = 0.01

# dram__bytes_read.sum + dram__bytes_write.sum of the dominant GEMM launch, from the ncu
# captures summarised under profiles/ (bytes per launch), keyed by (workload, rows per GPU).
# A GEMM's DRAM traffic depends on its shape, so other shapes report null rather than a
# scaled guess.
NCU_GEMM_TRAFFIC = {
    ("c4", 65536): {"bytes": 66.9e9,
                    "note": "forward 65536x8192x8192: 62.5 GB read + 4.36 GB written against 9.1 GB "
                            "compulsory, 270 GB/s = 4 % of HBM bandwidth (profiles/gemm_f64_tma_dmma_c4_traffic.md)"},
    ("c3", 8192): {"bytes": 2.06e9,
                   "note": "forward 8192x4096x4096: 1.80 GB read + 0.26 GB written against 0.67 GB compulsory "
                           "(profiles/gemm_f64_tma_dmma_c3.md)"},
}
SEED = 0
L2_BYTES = 126 << 20


def gemm_flops_per_sample(dims: list[int]) -> int:
    """forward + dW + dX for every Linear, minus the first layer's unused dX."""
    return sum(6 * a * b for a, b in zip(dims[:-1], dims[1:])) - 2 * dims[0] * dims[1]


def read_measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return {}


# --------------------------------------------------------------------------------------
# clocks during the timed region
# --------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.samples, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def top_up(self, keep_busy, min_samples: int = 3, limit_s: float = 3.0) -> None:
        """A timed region shorter than the 200 ms sampling period leaves no sample: keep the
        same load running (untimed) until a few have arrived, and say so in the record."""
        if self.proc is None or len(self.samples) >= min_samples:
            return
        self.topped_up = True
        t0 = time.perf_counter()
        while len(self.samples) < min_samples and time.perf_counter() - t0 < limit_s:
            keep_busy()

    def stop(self) -> dict:
        out = self._stop()
        out["sampled"] = ("under the same load directly after the timed region (it is shorter than the "
                          "sampling period)") if getattr(self, "topped_up", False) else "during the timed region"
        return out

    def _stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()          # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] or sm
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


# --------------------------------------------------------------------------------------
# the CPU arm (restatement of the reference, host cores)
# --------------------------------------------------------------------------------------
def cpu_sample_batch(workload: str) -> int:
    """Rows of the bounded CPU sample: a few seconds of work per step on a server CPU."""
    return {"c1": 32, "c2": 4096, "c3": 512, "c4": 64}[workload]


def run_cpu_steps(workload: str, steps: int, warmup: int, threads: int | None = None):
    """Times `steps` training steps of the workload's network on the host cores at a
    reduced batch (the sample).  Returns (samples/s, description, threads)."""
    from oracle import oracle_c as oc
    from rstorch_b200 import synth
    dims, _, stream, _ = WORKLOADS[workload]
    batch = cpu_sample_batch(workload)
    if threads:
        oc.set_threads(threads)
    threads = oc.max_threads()
    weights = synth.mlp_weights(SEED, dims)
    total = batch * (steps + warmup)
    if stream == "mnist_like":
        X, T = synth.mnist_like(SEED, 0, total)
    else:
        X, T = synth.gaussian_batch(SEED, 0, 0, total, dims[0], dims[-1], total)
    if warmup:
        oc.mlp_train(dims, weights, X, T, batch, warmup, LR, skip_first_dx=True, want_grads=False)
    t0 = time.perf_counter()
    oc.mlp_train(dims, weights, X[warmup * batch:], T[warmup * batch:], batch, steps, LR,
                 skip_first_dx=True, want_grads=False)
    dt = time.perf_counter() - t0
    what = f"{steps} step(s) of the same network at batch {batch} on {threads} host thread(s)"
    return batch * steps / dt, what, threads, dt / steps * 1e3


def run_cpu_sgd(steps: int, numel: int, threads: int | None = None):
    from oracle import oracle_c as oc
    from rstorch_b200 import synth
    if threads:
        oc.set_threads(threads)
    threads = oc.max_threads()
    p = synth.normal(synth.stream_key(SEED, "sgd.p"), numel, std=0.02)
    g = synth.normal(synth.stream_key(SEED, "sgd.g"), numel, std=1e-3)
    import ctypes as C
    lib = oc.load()
    pp, gp = p.ctypes.data_as(oc.PD), g.ctypes.data_as(oc.PD)
    lib.orc_sgd_step(pp, gp, C.c_int64(numel), C.c_double(LR))
    t0 = time.perf_counter()
    for _ in range(steps):
        lib.orc_sgd_step(pp, gp, C.c_int64(numel), C.c_double(LR))
    dt = time.perf_counter() - t0
    return numel * steps / dt, f"{steps} pass(es) over {numel} parameters on {threads} host thread(s)", threads, dt / steps * 1e3


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = args.workload
    if wl == "c5":
        value, what, threads, ms = run_cpu_sgd(args.steps, 1 << 26)
        metric, unit = "SGD parameters/sec", "params/s"
    else:
        value, what, threads, ms = run_cpu_steps(wl, args.steps, args.warmup)
        metric, unit = "train samples/sec (fwd+bwd+SGD)", "samples/s"
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES[wl], "lr": LR,
                   "note": "CPU restatement of the reference (the Rust crate cannot be built here); "
                           "each step is a bounded sample of the workload"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": what},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
def init_distributed(n: int):
    """(rank, world, local_rank, dist or None).  One process per GPU under torchrun."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1:
        return 0, 1, 0, None
    import torch
    import torch.distributed as dist
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    return rank, world, local, dist


def barrier_all(dist, ctx):
    ctx.synchronize()
    if dist is not None:
        import torch
        dist.barrier()
        torch.cuda.synchronize()


def max_over_ranks(dist, value: float) -> float:
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def build_model(rt, ctx, dims, identity):
    from rstorch_b200 import synth

    class Injected(rt.InitParameters):
        def __init__(self, w, b):
            self.w, self.b = w, b

        def weight(self, i, o):
            return self.w

        def bias(self, i, o):
            return self.b

    layers = [rt.Identity()] if identity else []
    n = len(dims) - 1
    for l in range(n):
        w, b = synth.mlp_weights_layer(SEED, dims, l)
        lin = rt.Linear.new_with_kernel(dims[l], dims[l + 1], Injected(w, b), ctx)
        lin._host_weight = lin._host_bias = None      # the host copy is not needed again
        layers.append(lin)
        if l + 1 < n:
            layers.append(rt.ReLU())
    return rt.sequential(*layers)


def mlp_arm(args) -> None:
    import rstorch_b200 as rt
    from rstorch_b200 import synth
    rank, world, local, dist = init_distributed(args.gpus)
    wl = args.workload
    dims, global_batch, stream, identity = WORKLOADS[wl]
    if args.batch:
        global_batch = args.batch
    first_row, rows = rt.shard_rows(global_batch, rank, world)
    ctx = rt.Context(local)
    comm = rt.Communicator.from_torch_distributed(ctx) if dist is not None else None
    model = build_model(rt, ctx, dims, identity)
    loss_fn, optim = rt.CrossEntropyLoss(), rt.SGD.new(LR)
    features, classes = dims[0], dims[-1]

    # two distinct resident batches (device leg) that are also the pinned host batches (e2e leg)
    n_batches = 2
    ds_x = np.empty((n_batches * rows, features))
    ds_t = np.empty((n_batches * rows, classes))
    for k in range(n_batches):
        if stream == "mnist_like":
            x, t = synth.mnist_like(SEED, k * global_batch + first_row, rows)
        else:
            x, t = synth.gaussian_batch(SEED, k, first_row, rows, features, classes, global_batch)
        ds_x[k * rows:(k + 1) * rows], ds_t[k * rows:(k + 1) * rows] = x, t
    resident = [(ctx.tensor(ds_x[k * rows:(k + 1) * rows]), ctx.tensor(ds_t[k * rows:(k + 1) * rows]))
                for k in range(n_batches)]

    def step(x, t, slot):
        pred = model.forward(x)
        loss_fn.forward_async(pred, t, slot)
        rt.backward_with_exchange(model, loss_fn.backward(), comm, need_input_grad=False)
        optim.step(model)

    input_bytes = rows * (features + classes) * 8
    flush = input_bytes < 2 * L2_BYTES           # small working set: flush L2 between timed steps
    use_graph = flush and comm is None           # launch-bound configurations replay a CUDA graph
    timer = ctx.timer()

    # ---- device-resident leg ----------------------------------------------------------
    graphs = None
    for w in range(max(args.warmup, 3)):
        step(*resident[w % n_batches], 0)
    if use_graph:
        graphs = []
        for k in range(n_batches):
            with ctx.capture() as cap:
                step(*resident[k], k)
            graphs.append(cap.graph)
        for k in range(n_batches):
            graphs[k].launch()
    loss_fn.result(0)
    sampler = ClockSampler(local)
    barrier_all(dist, ctx)
    sampler.start()
    launches0 = ctx.launch_count()
    total_ms = 0.0
    if flush:
        for k in range(args.steps):
            ctx.flush_l2(2 * L2_BYTES)
            timer.start()
            if graphs:
                graphs[k % n_batches].launch()
            else:
                step(*resident[k % n_batches], k % n_batches)
            timer.stop()
            total_ms += timer.elapsed_ms()
        launches = ctx.launch_count() - launches0 - args.steps          # minus the flush kernels
    else:
        timer.start()
        for k in range(args.steps):
            step(*resident[k % n_batches], k % n_batches)
        timer.stop()
        total_ms = timer.elapsed_ms()
        launches = ctx.launch_count() - launches0
    final_loss, final_acc = loss_fn.result((args.steps - 1) % n_batches)

    burst = max(1, min(200, int(150.0 / max(total_ms / args.steps, 1e-3))))     # about 150 ms of steps

    def same_load():
        for k in range(burst):
            if graphs:
                graphs[k % n_batches].launch()
            else:
                step(*resident[k % n_batches], k % n_batches)
        ctx.synchronize()

    if total_ms < 1000.0:
        sampler.top_up(same_load)
    barrier_all(dist, ctx)
    clocks = sampler.stop()
    total_ms = max_over_ranks(dist, total_ms)
    ms_per_step = total_ms / args.steps
    value = global_batch * args.steps / (total_ms * 1e-3)

    # ---- one instrumented step: device time per kernel class ---------------------------
    ctx.profile_begin()
    step(*resident[0], 0)
    prof = ctx.profile_end()
    gemm_ms = sum(ms for name, (cnt, ms) in prof.items() if name.startswith("gemm_"))
    gemm_launches = sum(cnt for name, (cnt, ms) in prof.items() if name.startswith("gemm_"))
    flops_step_local = gemm_flops_per_sample(dims) * rows

    # ---- end-to-end leg: host batches -> pinned ring -> step -> loss read back ---------
    ds = rt.ArrayDataset(ds_x, ds_t)
    loader = rt.DataLoader(ds, rows, False, rt.SequentialSampler(len(ds)), ctx, slots=2)
    loader._ensure_stager()
    for k in range(n_batches):                     # fill the pinned slots once, outside the timed region
        x_host, t_host = loader._host_views(k)
        x_host[...] = ds_x[k * rows:(k + 1) * rows]
        t_host[...] = ds_t[k * rows:(k + 1) * rows]
    del ds_x, ds_t
    lib = ctx._lib

    e2e_graphs = {}

    def e2e_step(k, read=True):
        slot = k % n_batches
        x, t = loader._acquire(slot)
        ctx._check(lib.rst_stager_submit(loader._stager, (k + 1) % n_batches))   # next batch's H2D overlaps this step
        if slot in e2e_graphs:
            e2e_graphs[slot].launch()               # the step on this slot's device tensors, replayed
        else:
            step(x, t, slot)
        return loss_fn.result(slot) if read else None

    ctx._check(lib.rst_stager_submit(loader._stager, 0))
    for k in range(2):
        e2e_step(k)
    if use_graph:
        # launch-bound workloads: one captured step per staging slot (its input tensors are fixed)
        for k in range(2, 2 + n_batches):
            slot = k % n_batches
            x, t = loader._acquire(slot)
            ctx._check(lib.rst_stager_submit(loader._stager, (k + 1) % n_batches))
            with ctx.capture() as cap:
                step(x, t, slot)
            e2e_graphs[slot] = cap.graph
            cap.graph.launch()
            loss_fn.result(slot)
    barrier_all(dist, ctx)
    t0 = time.perf_counter()
    timer.start()
    for k in range(2, 2 + args.steps):
        e2e_step(k)                                 # blocks on this step's loss, like `loss.forward -> f64`
    timer.stop()
    e2e_ms = max(timer.elapsed_ms(), (time.perf_counter() - t0) * 1e3)
    barrier_all(dist, ctx)
    e2e_ms = max_over_ranks(dist, e2e_ms)
    e2e_value = global_batch * args.steps / (e2e_ms * 1e-3)

    # ---- end-to-end with the u8 dataset resident in HBM (MNIST-shaped workloads) --------
    # The per-step host traffic is the batch's sample indices; gather, normalise, flatten
    # and one-hot run in one kernel on the device.
    e2e_device = None
    if stream == "mnist_like" and dist is None:
        n_samples = rows * 8
        images, labels = synth.mnist_like_u8(SEED, 0, n_samples)
        dds = rt.DeviceDataset(ctx, images, labels, classes)
        # The whole step, batch transform included, is one captured graph: per step the host
        # writes the sample indices into the dataset's pinned index stage and replays it.
        xg, tg = ctx.empty(rows, dims[0]), ctx.empty(rows, classes)
        stage = dds.index_stage(rows)
        order = np.arange(n_samples, dtype=np.int64)          # sequential sampler, no shuffle
        stage[:] = order[:rows]
        dds.gather_staged(rows, xg, tg)
        step(xg, tg, 0)
        loss_fn.result(0)
        with ctx.capture() as cap:
            dds.gather_staged(rows, xg, tg)
            step(xg, tg, 0)
        dataset_graph = cap.graph

        def run_epochs(n_steps):
            for k in range(n_steps):
                b = k % (n_samples // rows)
                stage[:] = order[b * rows:(b + 1) * rows]
                dataset_graph.launch()
                loss_fn.result(0)                 # blocks: the stage is free for the next indices

        run_epochs(3)
        ctx.synchronize()
        t0 = time.perf_counter()
        timer.start()
        run_epochs(args.steps)
        timer.stop()
        dev_ms = max(timer.elapsed_ms(), (time.perf_counter() - t0) * 1e3)
        e2e_device = {"value": global_batch * args.steps / (dev_ms * 1e-3), "unit": "samples/s",
                      "h2d_bytes_per_step": rows * 8, "d2h_bytes_per_step": 32,
                      "ms_per_step": dev_ms / args.steps,
                      "note": "u8 dataset resident in HBM; gather/normalise/one-hot kernel and the step "
                              "replayed as one graph, sample indices through the pinned index stage"}
    ctx.check_device()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel --------------------------------------------------
    peaks = read_measured_peaks()
    fp64_peak = ctx.probe_fp64_peak(0, 2048)
    achieved = flops_step_local / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    traffic = NCU_GEMM_TRAFFIC.get((wl, rows))
    roofline = {
        "bound": "tensor", "kernel": "gemm_f64_tma_dmma",
        "achieved": achieved, "peak": fp64_peak, "unit": "TFLOP/s",
        "frac": achieved / fp64_peak if achieved else None,
        "traffic": traffic["bytes"] if traffic else None,
        "traffic_note": traffic["note"] if traffic else "no ncu capture at this shape",
        "peak_source": "f64 DMMA issue-rate probe run in this process (MEASURED_PEAKS.json records no f64 "
                       "figure; its bf16 peak does not bound an f64 kernel)",
        "launches_per_step": gemm_launches, "kernel_ms_per_step": gemm_ms,
        "step_tflops": flops_step_local * world / (ms_per_step * 1e-3) / 1e12,
    }
    line = {
        "metric": "train samples/sec (fwd+bwd+SGD)", "value": value, "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES[wl], "layers": dims, "global_batch": global_batch,
                   "rows_per_gpu": rows, "lr": LR, "parallelism": f"dp{world}",
                   "l2": "flushed between timed steps" if flush else "inputs larger than L2",
                   "graph_replay": bool(graphs), "first_layer_dx": "skipped",
                   "final_loss": final_loss, "final_accuracy": final_acc},
        "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": input_bytes,
                "d2h_bytes_per_step": 32, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
        "kernel_classes_ms": {k: round(v[1], 4) for k, v in prof.items()},
        "hbm_peak_gbs_measured": peaks.get("hbm_gbs"),
    }
    if e2e_device is not None:
        line["e2e_device_dataset"] = e2e_device
    if world == 1:
        cpu_value, what, threads, _ = run_cpu_steps(wl, 1, 0)
        line["cpu_baseline"] = {"value": cpu_value, "unit": "samples/s", "cores": threads, "kind": "port",
                                "sample": what}
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


def sgd_arm(args) -> None:
    """Workload c5: the fused SGD step alone over 2^30 parameters in 64 tensors,
    parameter range split evenly over the ranks (no communication)."""
    import rstorch_b200 as rt
    from rstorch_b200 import synth
    from rstorch_b200.core import handle_array
    rank, world, local, dist = init_distributed(args.gpus)
    ctx = rt.Context(local)
    total = (1 << args.sgd_log2_params) // world
    sizes = synth.sgd_tensor_sizes(SEED + rank, total, 64)
    params, grads = [], []
    chunk = np.empty(max(sizes))
    for i, n in enumerate(sizes):
        p, g = ctx.empty(1, n), ctx.empty(1, n)
        p.upload(synth.normal(synth.stream_key(SEED, "sgd.p", rank * 64 + i), n, std=0.02, out=chunk[:n]))
        g.upload(synth.normal(synth.stream_key(SEED, "sgd.g", rank * 64 + i), n, std=1e-3, out=chunk[:n]))
        params.append(p); grads.append(g)
    pa, ga = handle_array(params), handle_array(grads)
    lib = ctx._lib

    def step():
        ctx._check(lib.rst_sgd_step(ctx.handle, len(params), pa, ga, LR))

    for _ in range(max(args.warmup, 3)):
        step()
    timer = ctx.timer()
    sampler = ClockSampler(local)
    barrier_all(dist, ctx)
    sampler.start()
    launches0 = ctx.launch_count()
    timer.start()
    for _ in range(args.steps):
        step()
    timer.stop()
    total_ms = timer.elapsed_ms()
    launches = ctx.launch_count() - launches0

    def same_load():
        for _ in range(max(1, min(200, int(150.0 * args.steps / max(total_ms, 1e-3))))):
            step()
        ctx.synchronize()

    if total_ms < 1000.0:
        sampler.top_up(same_load)
    barrier_all(dist, ctx)
    clocks = sampler.stop()
    total_ms = max_over_ranks(dist, total_ms)
    ms = total_ms / args.steps
    numel = total * world
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peaks = read_measured_peaks()
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    achieved = 24.0 * total / (ms * 1e-3) / 1e9
    line = {
        "metric": "SGD parameters/sec", "value": numel / (ms * 1e-3), "unit": "params/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES["c5"], "tensors_per_gpu": 64, "params_per_gpu": total, "lr": LR,
                   "l2": "inputs larger than L2"},
        "e2e": None, "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "sgd_multi_tensor_kernel", "achieved": achieved, "peak": hbm_peak,
                     "unit": "GB/s", "frac": achieved / hbm_peak,
                     # ncu on a 2^27-parameter launch: 3.18 GB moved against 3.22 GB algorithmic; an
                     # elementwise kernel's traffic grows in proportion to the parameter count
                     "traffic": 24.0 * total * (3.184 / 3.221),
                     "traffic_note": "scaled from the 2^27-parameter capture in profiles/sgd_multi_tensor_kernel_c5.md",
                     "peak_source": "MEASURED_PEAKS.json hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650",
                     "frac_of_nominal_8000": achieved / 8000.0},
    }
    if world == 1:
        v, what, threads, _ = run_cpu_sgd(2, 1 << 26)
        line["cpu_baseline"] = {"value": v, "unit": "params/s", "cores": threads, "kind": "port", "sample": what}
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


def emit(line: dict) -> None:
    """One JSON line; non-finite floats become null so that the line stays valid JSON."""
    def clean(v):
        if isinstance(v, float) and not np.isfinite(v):
            return None
        if isinstance(v, dict):
            return {k: clean(x) for k, x in v.items()}
        if isinstance(v, (list, tuple)):
            return [clean(x) for x in v]
        if isinstance(v, (np.floating, np.integer)):
            return clean(v.item())
        return v
    print(json.dumps(clean(line)), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOAD_NAMES), default="c4")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the workload's global batch (profiler captures and parity runs; "
                         "the benchmark numbers use the workload's own batch)")
    ap.add_argument("--sgd-log2-params", type=int, default=30,
                    help="workload c5 only: log2 of the parameter count (30 is the benchmark size; "
                         "smaller values are for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload == "c5":
        sgd_arm(args)
    else:
        mlp_arm(args)


if __name__ == "__main__":
    main()
