#!/usr/bin/env python
"""Benchmark of the f64 training step (forward + loss + backward [+ all-reduce] + SGD).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5]
                    [--impl ours|reference]

Prints ONE JSON line.  The default workload is the deep MLP that the headline
metric is quoted on at 1/2/4/8 GPUs: 4096 -> 8192 -> 8 x (8192 -> 8192) -> 1000
(10 Linear layers, ReLU between them), f64, global batch 65536 split evenly over
the ranks (strong scaling), SGD lr 0.01, gradients averaged with NCCL before the
single-launch SGD step.  Inputs are seeded synthetic data of that shape.

`value` times the step with the batch already in HBM.  `e2e` times the same step
fed through `DataLoader.iter_array()`: the rows of every batch are gathered into a
pinned slot on the host, copied to the device and the step's loss is read back,
all inside the timed region.  `verify` (outside the timed regions) recomputes
sampled entries of the benched GEMM shapes on the host in long double, compares the
replicas' weights bit for bit and reports the loss averaged over all ranks.
With the default workload the line also carries short legs of the other workloads
(`other_workloads`).  `--impl reference` times the CPU restatement of the
reference's step on the host cores (the reference itself is Rust over un-vendored
crates and cannot be built with the toolchains of this image).
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

# dram__bytes_read.sum + dram__bytes_write.sum of the dominant GEMM launch, from ncu
# captures (bytes per launch), keyed by (workload, rows per GPU).  A GEMM's DRAM traffic
# depends on its shape, so other shapes report null rather than a scaled guess.
NCU_GEMM_TRAFFIC = {
    ("c4", 65536): {"bytes": 66.9e9,
                    "note": "ncu capture of forward 65536x8192x8192: 62.5 GB read + 4.36 GB written against "
                            "9.1 GB compulsory, 270 GB/s = 4 % of HBM bandwidth"},
    ("c3", 8192): {"bytes": 2.06e9,
                   "note": "ncu capture of forward 8192x4096x4096: 1.80 GB read + 0.26 GB written against "
                           "0.67 GB compulsory"},
}
SEED = 0
L2_BYTES = 126 << 20
E2E_SLOTS = 3


def gemm_flops_per_sample(dims: list[int]) -> int:
    """forward + dW + dX for every Linear, minus the first layer's unused dX."""
    return sum(6 * a * b for a, b in zip(dims[:-1], dims[1:])) - 2 * dims[0] * dims[1]


def read_measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return {}


def host_threads() -> int:
    """Hardware threads this process may run on, whatever OMP_NUM_THREADS says (a launcher
    such as torch.distributed.run sets it to 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


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
# the CPU arm (restatement of the reference, host cores).  Nothing below this header and
# above "our arm" touches the CUDA library: inputs come from the oracle's own generator.
# --------------------------------------------------------------------------------------
CPU_SAMPLE_ROWS = {"c1": 32, "c2": 4096, "c3": 512, "c4": 256}          # all host threads
CPU_SAMPLE_ROWS_1THREAD = {"c1": 32, "c2": 4096, "c3": 128, "c4": 64}   # one thread, one step


class CpuArm:
    """The workload's network on the host cores at a reduced batch (the bounded sample):
    weights and batches from the oracle's generator (bit-identical to the GPU arm's)."""

    def __init__(self, workload: str):
        from oracle import oracle_c, oracle_synth
        self.oc, self.synth, self.wl = oracle_c, oracle_synth, workload
        self.dims, _, self.stream, _ = WORKLOADS[workload]
        self.oc.set_threads(host_threads())
        self.weights = self.synth.mlp_weights(SEED, self.dims)

    def _batches(self, rows: int, steps: int):
        total = rows * steps
        if self.stream == "mnist_like":
            return self.synth.mnist_like(SEED, 0, total)
        return self.synth.gaussian_batch(SEED, 0, 0, total, self.dims[0], self.dims[-1], total)

    def run(self, steps: int, warmup: int, threads: int, rows: int):
        """(samples/s, ms per step, threads used, description); weights keep training on."""
        self.oc.set_threads(threads)
        used = self.oc.max_threads()
        X, T = self._batches(rows, steps + warmup)
        if warmup:
            self.oc.mlp_train(self.dims, self.weights, X, T, rows, warmup, LR, skip_first_dx=True, want_grads=False)
        t0 = time.perf_counter()
        self.oc.mlp_train(self.dims, self.weights, X[warmup * rows:], T[warmup * rows:], rows, steps, LR,
                          skip_first_dx=True, want_grads=False)
        dt = time.perf_counter() - t0
        what = f"{steps} step(s) of the same network at batch {rows} on {used} host thread(s)"
        return rows * steps / dt, dt / steps * 1e3, used, what

    def baseline(self, steps: int, warmup: int) -> dict:
        """All host threads, then one thread (the reference enables no threading,
        Cargo.toml:16-21, so the single-thread figure is the one faithful to it)."""
        value, ms, used, what = self.run(steps, warmup, host_threads(), CPU_SAMPLE_ROWS[self.wl])
        v1, _, _, what1 = self.run(1, 0, 1, CPU_SAMPLE_ROWS_1THREAD[self.wl])
        self.oc.set_threads(host_threads())
        return {"value": value, "unit": "samples/s", "cores": used, "kind": "port", "sample": what,
                "ms_per_step": ms, "value_1thread": v1, "sample_1thread": what1,
                "inputs": "oracle generator (bit-identical to the GPU arm's streams)"}


def cpu_sgd(steps: int, numel: int, threads: int):
    from oracle import oracle_c as oc
    from oracle import oracle_synth as osy
    import ctypes as C
    oc.set_threads(threads)
    used = oc.max_threads()
    p = osy.normal(osy.stream_key(SEED, "sgd.p"), numel, std=0.02)
    g = osy.normal(osy.stream_key(SEED, "sgd.g"), numel, std=1e-3)
    lib = oc.load()
    pp, gp = p.ctypes.data_as(oc.PD), g.ctypes.data_as(oc.PD)
    lib.orc_sgd_step(pp, gp, C.c_int64(numel), C.c_double(LR))
    t0 = time.perf_counter()
    for _ in range(steps):
        lib.orc_sgd_step(pp, gp, C.c_int64(numel), C.c_double(LR))
    dt = time.perf_counter() - t0
    return numel * steps / dt, dt / steps * 1e3, used, f"{steps} pass(es) over {numel} parameters on {used} host thread(s)"


def cpu_sgd_baseline(steps: int) -> dict:
    v, ms, used, what = cpu_sgd(steps, 1 << 26, host_threads())
    v1, _, _, what1 = cpu_sgd(1, 1 << 26, 1)
    return {"value": v, "unit": "params/s", "cores": used, "kind": "port", "sample": what, "ms_per_step": ms,
            "value_1thread": v1, "sample_1thread": what1}


def reference_arm(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    wl = args.workload
    if wl == "c5":
        base = cpu_sgd_baseline(args.steps)
        metric = "SGD parameters/sec"
    else:
        base = CpuArm(wl).baseline(args.steps, args.warmup)
        metric = "train samples/sec (fwd+bwd+SGD)"
    line = {
        "impl": "reference", "metric": metric, "value": base["value"], "unit": base["unit"], "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES[wl], "lr": LR,
                   "note": "CPU restatement of the reference (the Rust crate cannot be built here); each step is "
                           "a bounded sample of the workload; the thread count is set by this program and does "
                           "not follow OMP_NUM_THREADS"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": base["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
class Env:
    """One process = one rank = one GPU."""

    def __init__(self, n: int):
        import rstorch_b200 as rt
        self.rt = rt
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank, self.local, self.dist = 0, 0, None
        if self.world > 1:
            import torch
            import torch.distributed as dist
            self.rank = int(os.environ["RANK"])
            self.local = int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
            torch.cuda.set_device(self.local)
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", rank=self.rank, world_size=self.world,
                                    device_id=torch.device("cuda", self.local))
            self.dist = dist
        self.ctx = rt.Context(self.local)
        self.comm = rt.Communicator.from_torch_distributed(self.ctx) if self.dist is not None else None

    def barrier(self):
        self.ctx.synchronize()
        if self.dist is not None:
            import torch
            self.dist.barrier()
            torch.cuda.synchronize()

    def reduce(self, value: float, op: str = "max") -> float:
        if self.dist is None:
            return value
        import torch
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        self.dist.all_reduce(t, op={"max": self.dist.ReduceOp.MAX, "sum": self.dist.ReduceOp.SUM}[op])
        return float(t.item())

    def gather_u64(self, values: list[int]) -> list[list[int]]:
        """Every rank's list of 64-bit words, on every rank."""
        if self.dist is None:
            return [values]
        import torch
        mine = torch.tensor(np.array(values, dtype=np.uint64).view(np.int64), device="cuda")
        out = [torch.empty_like(mine) for _ in range(self.world)]
        self.dist.all_gather(out, mine)
        return [[int(v) & 0xFFFFFFFFFFFFFFFF for v in o.cpu().tolist()] for o in out]

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


class CyclingSampler:
    """Sampler indices 0, 1, ..., n-1, 0, 1, ... (`total` of them): an epoch of `total /
    batch` batches over a dataset that holds a few distinct batches."""

    def __init__(self, n: int, total: int):
        self.n, self.size = int(n), int(total)

    def iter(self):
        return iter(np.arange(self.size, dtype=np.int64) % self.n)


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


def verify_benched_shapes(env: Env, model, x_resident, samples: int = 64) -> dict:
    """Sampled entries of the GEMM shapes the timed step runs, against long-double dot
    products on the host.  The layer is the second Linear of the network with its current
    weights; its input is the activation the model computes for a resident batch; the
    incoming gradient is a seeded N(0,1) matrix.  Forward (bias + ReLU epilogue), dW (K =
    rows of this rank), dX through the transposed-companion kernel with the ReLU mask, the
    transposed copy that kernel stores, and db are all checked."""
    from rstorch_b200 import synth
    rt, ctx = env.rt, env.ctx
    lins = [l for l in model.layers if isinstance(l, rt.Linear)]
    lin = lins[1] if len(lins) > 2 else lins[0]
    model.forward(x_resident)                         # leaves every layer's cached input in place
    X = lin.prev_input                                # (rows, in): post-ReLU output of the layer in front
    nxt = lins[lins.index(lin) + 1]
    Y = nxt.prev_input                                # (rows, out) = max(X·Wᵀ + b, 0)
    rows, cin, cout = X.rows, lin.input_size, lin.output_size
    lib = ctx._lib
    Xt, Yt = ctx.empty(cin, rows), None
    ctx._check(lib.rst_transpose(ctx.handle, X.handle, Xt.handle))
    dY_host = synth.normal(synth.stream_key(SEED, "verify.dY", env.rank), rows * cout).reshape(rows, cout)
    dY = ctx.tensor(dY_host)
    del dY_host
    dYt = ctx.empty(cout, rows)
    ctx._check(lib.rst_transpose(ctx.handle, dY.handle, dYt.handle))
    dW, db = ctx.empty(cout, cin), ctx.empty(1, cout)
    dX, dXt = ctx.empty(rows, cin), ctx.empty(cin, rows)
    ctx._check(lib.rst_linear_backward_t(ctx.handle, dY.handle, dYt.handle, X.handle, lin.weight.handle, X.handle,
                                         dW.handle, db.handle, dX.handle, dXt.handle))
    W = lin.weight.numpy()
    b = lin.bias.numpy().reshape(-1)
    ld = np.longdouble
    # ranks that exchange shares of the global-batch gradient divide by all ranks' rows
    grad_rows = rows * (env.world if (env.comm is not None and getattr(env.comm, "shares", False)) else 1)
    rng = np.random.default_rng(1234 + env.rank)

    def row(t, r):                                    # row r of a device matrix, 8·cols bytes over the bus
        return t.slice(r * t.cols, 1, t.cols).numpy().reshape(-1)

    err = {"forward": 0.0, "dW": 0.0, "dX": 0.0, "db": 0.0}
    scale = {"forward": 0.0, "dW": 0.0, "dX": 0.0}
    diffs = {"forward": [], "dW": [], "dX": []}
    dxt_equal = True
    for _ in range(samples):
        r, c, k = int(rng.integers(0, rows)), int(rng.integers(0, cout)), int(rng.integers(0, cin))
        x_r, dy_r = row(X, r), row(dY, r)
        want_y = max(float(np.dot(x_r.astype(ld), W[c].astype(ld)) + ld(b[c])), 0.0)
        got_y = float(row(Y, r)[c])
        want_dx = float(np.dot(dy_r.astype(ld), W[:, k].astype(ld))) * (1.0 if x_r[k] > 0.0 else 0.0)
        got_dx = float(row(dX, r)[k])
        dxt_equal = dxt_equal and float(row(dXt, k)[r]) == got_dx
        want_dw = float(np.dot(row(dYt, c).astype(ld), row(Xt, k).astype(ld)) / ld(grad_rows))
        got_dw = float(row(dW, c)[k])
        for name, got, want in (("forward", got_y, want_y), ("dX", got_dx, want_dx), ("dW", got_dw, want_dw)):
            diffs[name].append(abs(got - want))
            scale[name] = max(scale[name], abs(want))
    for name in diffs:
        err[name] = max(diffs[name]) / scale[name] if scale[name] > 0 else max(diffs[name])
    db_host = db.numpy().reshape(-1)
    cols = rng.integers(0, cout, size=8)
    want_db = np.array([float(row(dYt, int(c)).astype(ld).sum() / ld(grad_rows)) for c in cols])
    err["db"] = float(np.max(np.abs(db_host[cols] - want_db)) / max(np.max(np.abs(want_db)), 1e-300))
    ctx.check_device()
    return {"layer": f"Linear({cin}, {cout}) at {rows} rows", "sampled_entries_each": samples,
            "max_rel_err": max(err.values()), "rel_err": err,
            "formula": "max|gpu - long double| / max|long double| over the sampled entries of each product",
            "transposed_copy_equals_dX": bool(dxt_equal)}


def run_mlp_workload(env: Env, wl: str, steps: int, warmup: int, batch: int = 0, verify: bool = True) -> dict:
    """Resident leg, per-kernel-class timing, end-to-end leg (and, for the headline run, the
    verify block) of one MLP workload.  Every large object is local, so it is gone when
    the function returns."""
    from rstorch_b200 import synth
    rt, ctx, comm, dist, rank, world = env.rt, env.ctx, env.comm, env.dist, env.rank, env.world
    dims, global_batch, stream, identity = WORKLOADS[wl]
    if batch:
        global_batch = batch
    first_row, rows = rt.shard_rows(global_batch, rank, world)
    model = build_model(rt, ctx, dims, identity)
    loss_fn, optim = rt.CrossEntropyLoss(), rt.SGD.new(LR)
    features, classes = dims[0], dims[-1]
    warmup = max(warmup, 3)

    # two distinct batches: resident on the device (device leg) and rows of the host dataset (e2e leg)
    n_batches = 2
    ds_x = np.empty((n_batches * rows, features))
    ds_t = np.empty((n_batches * rows, classes))
    for k in range(n_batches):
        if stream == "mnist_like":
            x, t = synth.mnist_like(SEED, k * global_batch + first_row, rows)
        else:
            x, t = synth.gaussian_batch(SEED, k, first_row, rows, features, classes, global_batch)
        ds_x[k * rows:(k + 1) * rows], ds_t[k * rows:(k + 1) * rows] = x, t
    del x, t
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
    for w in range(warmup):
        step(*resident[w % n_batches], 0)
    if use_graph:
        graphs = []
        for k in range(n_batches):
            step(*resident[k], k)                  # the unrecorded run that fills the allocator's cache
            with ctx.capture() as cap:
                step(*resident[k], k)
            graphs.append(cap.graph)
        for k in range(n_batches):
            graphs[k].launch()
    loss_fn.result(0)
    sampler = ClockSampler(env.local)
    env.barrier()
    sampler.start()
    launches0 = ctx.launch_count()
    total_ms = 0.0
    if flush:
        for k in range(steps):
            ctx.flush_l2(2 * L2_BYTES)
            timer.start()
            if graphs:
                graphs[k % n_batches].launch()
            else:
                step(*resident[k % n_batches], k % n_batches)
            timer.stop()
            total_ms += timer.elapsed_ms()
        launches = ctx.launch_count() - launches0 - steps          # minus the flush kernels
    else:
        timer.start()
        for k in range(steps):
            step(*resident[k % n_batches], k % n_batches)
        timer.stop()
        total_ms = timer.elapsed_ms()
        launches = ctx.launch_count() - launches0
    final_loss, final_acc = loss_fn.result((steps - 1) % n_batches)

    burst = max(1, min(200, int(150.0 / max(total_ms / steps, 1e-3))))     # about 150 ms of steps

    def same_load():
        for k in range(burst):
            if graphs:
                graphs[k % n_batches].launch()
            else:
                step(*resident[k % n_batches], k % n_batches)
        ctx.synchronize()

    if total_ms < 1000.0:
        sampler.top_up(same_load)
    env.barrier()
    clocks = sampler.stop()
    total_ms = env.reduce(total_ms, "max")
    ms_per_step = total_ms / steps
    value = global_batch * steps / (total_ms * 1e-3)
    # the loss of the whole batch = the mean of the equal shards' means
    global_loss = env.reduce(final_loss, "sum") / world
    global_acc = env.reduce(final_acc, "sum") / world

    # ---- one instrumented step: device time per kernel class ---------------------------
    ctx.profile_begin()
    step(*resident[0], 0)
    prof = ctx.profile_end()
    gemm_ms = sum(ms for name, (cnt, ms) in prof.items() if name.startswith("gemm_"))
    gemm_launches = sum(cnt for name, (cnt, ms) in prof.items() if name.startswith("gemm_"))
    flops_step_local = gemm_flops_per_sample(dims) * rows

    # ---- evidence, outside every timed region --------------------------------------------
    verify_block = None
    if verify:
        digests = [p.parm.checksum() for p in model.parameters()]
        per_rank = env.gather_u64(digests)
        verify_block = {"replicas_identical": all(r == per_rank[0] for r in per_rank),
                        "replica_digest": f"{(sum(per_rank[0]) & 0xFFFFFFFFFFFFFFFF):016x}",
                        "ranks_compared": len(per_rank),
                        "global_mean_loss": global_loss, "global_accuracy": global_acc}
        if len(dims) > 3 and min(dims[1:-1]) >= 1024:
            verify_block.update(verify_benched_shapes(env, model, resident[0][0]))
            worst = env.reduce(verify_block["max_rel_err"], "max")
            verify_block["max_rel_err"] = worst
        verify_block["within_1e-9"] = (verify_block.get("max_rel_err", 0.0) < 1e-9)
    if graphs:
        for g in graphs:
            g.destroy()
        graphs = None
    del resident

    # ---- end-to-end leg: host rows -> DataLoader.iter_array -> step -> loss read back -----
    # Large batches are assembled on the loader's helper thread (np.take into the pinned slot
    # overlaps the previous step); small ones inline, where a thread hand-over would cost
    # more than the copy.
    prefetch = input_bytes >= (1 << 20)
    # three slots keep batch k (compute), k+1 (copy) and k+2 (assembly) in flight; batches that
    # take longer to assemble than to train on get more slots, i.e. more assembling threads
    slots = E2E_SLOTS if (not prefetch or input_bytes >= (256 << 20)) else 2 * E2E_SLOTS
    e2e_warm = 2 * slots
    ds = rt.ArrayDataset(ds_x, ds_t)
    loader = rt.DataLoader(ds, rows, False, CyclingSampler(len(ds), rows * (steps + e2e_warm)), ctx,
                           slots=slots, prefetch=prefetch)
    e2e_graphs: dict[int, object] = {}
    batches = loader.iter_array()

    def e2e_step(k):
        x, t = next(batches)                      # batch k: assembled, copied, handed out by the loader
        slot = k % slots
        if slot in e2e_graphs:
            e2e_graphs[slot].launch()             # the step on this slot's device tensors, replayed
        else:
            step(x, t, slot)
            if use_graph:
                # launch-bound workloads: one recorded step per staging slot (its tensors are fixed)
                with ctx.capture() as cap:
                    step(x, t, slot)
                e2e_graphs[slot] = cap.graph
        return loss_fn.result(slot)               # blocks on this step's loss, like `loss.forward -> f64`

    for k in range(e2e_warm):
        e2e_step(k)
    env.barrier()
    t0 = time.perf_counter()
    timer.start()
    for k in range(e2e_warm, e2e_warm + steps):
        e2e_step(k)
    timer.stop()
    e2e_ms = max(timer.elapsed_ms(), (time.perf_counter() - t0) * 1e3)
    env.barrier()
    e2e_ms = env.reduce(e2e_ms, "max")
    e2e_value = global_batch * steps / (e2e_ms * 1e-3)
    batches.close()
    for g in e2e_graphs.values():
        g.destroy()
    loader.close()
    del ds, ds_x, ds_t

    # ---- end-to-end with the u8 dataset resident in HBM (MNIST-shaped workloads) --------
    # The per-step host traffic is the batch's sample indices; gather, normalise, flatten
    # and one-hot run in one kernel on the device.
    e2e_device = None
    if stream == "mnist_like" and dist is None:
        n_samples = rows * 8
        images, labels = synth.mnist_like_u8(SEED, 0, n_samples)
        dds = rt.DeviceDataset(ctx, images, labels, classes)
        # The whole step, batch transform included, is one recorded graph: per step the host
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
        run_epochs(steps)
        timer.stop()
        dev_ms = max(timer.elapsed_ms(), (time.perf_counter() - t0) * 1e3)
        e2e_device = {"value": global_batch * steps / (dev_ms * 1e-3), "unit": "samples/s",
                      "h2d_bytes_per_step": rows * 8, "d2h_bytes_per_step": 32,
                      "ms_per_step": dev_ms / steps,
                      "note": "u8 dataset resident in HBM; gather/normalise/one-hot kernel and the step "
                              "replayed as one graph, sample indices through the pinned index stage"}
        dataset_graph.destroy()
        dds.close()
    ctx.check_device()

    # ---- roofline of the dominant kernel --------------------------------------------------
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
    hbm = read_measured_peaks().get("hbm_gbs")
    if hbm and wl in ("c1", "c2"):
        # neither roofline bounds the launch-bound workloads: report both fractions, no target
        step_bytes = 3 * 8 * sum(a * b + b for a, b in zip(dims[:-1], dims[1:])) + 2 * input_bytes
        roofline["hbm_frac_of_measured"] = step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm
    out = {
        "metric": "train samples/sec (fwd+bwd+SGD)", "value": value, "unit": "samples/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES[wl], "layers": dims, "global_batch": global_batch,
                   "rows_per_gpu": rows, "lr": LR, "parallelism": f"dp{world}",
                   "l2": "flushed between timed steps" if flush else "inputs larger than L2",
                   "graph_replay": use_graph, "first_layer_dx": "skipped",
                   "final_loss": global_loss, "final_accuracy": global_acc,
                   "final_loss_is": "mean over all ranks of the last timed step's shard loss"},
        "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": input_bytes,
                "d2h_bytes_per_step": 32, "ms_per_step": e2e_ms / steps,
                "host_assembly": "inside the timed region: DataLoader.iter_array gathers every batch's rows "
                                 "into a pinned slot (" + (f"{slots - 2} helper thread(s), overlapping earlier steps"
                                                          if prefetch else "inline") + ")"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
        "kernel_classes_ms": {k: round(v[1], 4) for k, v in prof.items()},
    }
    if verify_block is not None:
        out["verify"] = verify_block
    if e2e_device is not None:
        out["e2e_device_dataset"] = e2e_device
    return out


def run_sgd_workload(env: Env, steps: int, warmup: int, log2_params: int = 30) -> dict:
    """Workload c5: the fused SGD step alone over 2^30 parameters in 64 tensors,
    parameter range split evenly over the ranks (no communication)."""
    from rstorch_b200 import synth
    from rstorch_b200.core import handle_array
    ctx, rank, world = env.ctx, env.rank, env.world
    total = (1 << log2_params) // world
    sizes = synth.sgd_tensor_sizes(SEED + rank, total, 64)
    params, grads = [], []
    chunk = np.empty(max(sizes))
    for i, n in enumerate(sizes):
        p, g = ctx.empty(1, n), ctx.empty(1, n)
        p.upload(synth.normal(synth.stream_key(SEED, "sgd.p", rank * 64 + i), n, std=0.02, out=chunk[:n]))
        g.upload(synth.normal(synth.stream_key(SEED, "sgd.g", rank * 64 + i), n, std=1e-3, out=chunk[:n]))
        params.append(p); grads.append(g)
    del chunk
    pa, ga = handle_array(params), handle_array(grads)
    lib = ctx._lib
    warmup = max(warmup, 3)

    def step():
        ctx._check(lib.rst_sgd_step(ctx.handle, len(params), pa, ga, LR))

    for _ in range(warmup):
        step()
    timer = ctx.timer()
    sampler = ClockSampler(env.local)
    env.barrier()
    sampler.start()
    launches0 = ctx.launch_count()
    timer.start()
    for _ in range(steps):
        step()
    timer.stop()
    total_ms = timer.elapsed_ms()
    launches = ctx.launch_count() - launches0

    def same_load():
        for _ in range(max(1, min(200, int(150.0 * steps / max(total_ms, 1e-3))))):
            step()
        ctx.synchronize()

    if total_ms < 1000.0:
        sampler.top_up(same_load)
    env.barrier()
    clocks = sampler.stop()
    total_ms = env.reduce(total_ms, "max")
    ms = total_ms / steps
    numel = total * world
    peaks = read_measured_peaks()
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    achieved = 24.0 * total / (ms * 1e-3) / 1e9
    ctx.check_device()
    return {
        "metric": "SGD parameters/sec", "value": numel / (ms * 1e-3), "unit": "params/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES["c5"] if log2_params == 30 else f"fused SGD step over 2^{log2_params} f64 parameters in 64 tensors",
                   "tensors_per_gpu": 64, "params_per_gpu": total, "lr": LR, "l2": "inputs larger than L2"},
        "e2e": None, "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "sgd_multi_tensor_kernel", "achieved": achieved, "peak": hbm_peak,
                     "unit": "GB/s", "frac": achieved / hbm_peak,
                     # ncu on a 2^27-parameter launch: 3.18 GB moved against 3.22 GB algorithmic; an
                     # elementwise kernel's traffic grows in proportion to the parameter count
                     "traffic": 24.0 * total * (3.184 / 3.221),
                     "traffic_note": "scaled from an ncu capture of a 2^27-parameter launch",
                     "peak_source": "MEASURED_PEAKS.json hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650",
                     "frac_of_nominal_8000": achieved / 8000.0},
    }


def brief(result: dict) -> dict:
    """The part of a workload's result that goes into `other_workloads`."""
    keep = ("metric", "value", "unit", "steps", "warmup", "ms_per_step", "gpu_launches", "clocks", "roofline",
            "e2e", "e2e_device_dataset", "scaling")
    out = {k: result[k] for k in keep if k in result}
    out["workload"] = result["config"]["workload"]
    if "verify" in result:
        out["verify"] = result["verify"]
    return out


def our_arm(args) -> None:
    env = Env(args.gpus)
    wl = args.workload
    if wl == "c5":
        line = run_sgd_workload(env, args.steps, args.warmup, args.sgd_log2_params)
    else:
        line = run_mlp_workload(env, wl, args.steps, args.warmup, args.batch)
    env.ctx.empty_cache()

    # Short legs of the other workloads ride along with the headline run, so that one
    # command measures them all; the headline keys above stay the requested workload's.
    if wl == "c4" and not args.batch and not args.no_other_workloads:
        others = {}
        if env.world == 1:
            others["c3"] = brief(run_mlp_workload(env, "c3", 20, 3))
            env.ctx.empty_cache()
        others["c5"] = brief(run_sgd_workload(env, 20, 3))
        env.ctx.empty_cache()
        if env.world == 1:
            others["c2"] = brief(run_mlp_workload(env, "c2", 200, 20))
            others["c1"] = brief(run_mlp_workload(env, "c1", 200, 20))
            env.ctx.empty_cache()
        line["other_workloads"] = others
    line["hbm_peak_gbs_measured"] = read_measured_peaks().get("hbm_gbs")

    if env.rank == 0 and env.world == 1:
        if wl == "c5":
            line["cpu_baseline"] = cpu_sgd_baseline(2)
        else:
            line["cpu_baseline"] = CpuArm(wl).baseline(1, 1)      # one untimed step first: thread pool, page faults
    if env.rank == 0:
        emit(line)
    env.close()


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
        if isinstance(v, np.bool_):
            return bool(v)
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
    ap.add_argument("--no-other-workloads", action="store_true",
                    help="with the default workload: skip the short legs of the other workloads")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        our_arm(args)


if __name__ == "__main__":
    main()
