"""The C++ façade (include/rstorch.hpp) over the C ABI: it compiles against the header
on any host, and on a GPU it re-runs the reference's unit tests and the README training
loop, whose trajectory is compared with the CPU restatement."""
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

from conftest import REL_TOL, ROOT, rel_err

SRC = os.path.join(ROOT, "tests", "cpp", "facade_tests.cpp")


def build(tmp_path) -> str:
    exe = str(tmp_path / "facade_tests")
    lib_dir = os.path.join(ROOT, "rstorch_b200")
    cmd = ["g++", "-std=c++17", "-O2", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
           SRC, "-L", lib_dir, "-lrstorch_b200", f"-Wl,-rpath,{lib_dir}", "-o", exe]
    env = dict(os.environ, CXX="g++")
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr
    return exe


def test_facade_compiles_against_the_header(tmp_path):
    exe = build(tmp_path)
    import torch
    if not torch.cuda.is_available():
        r = subprocess.run([exe], capture_output=True, text=True)
        assert r.returncode == 2 and "no CPU path" in r.stdout     # loud failure, no fallback


@pytest.mark.gpu
def test_reference_unit_tests_and_readme_loop_through_the_facade(tmp_path, oc):
    from rstorch_b200 import synth
    exe = build(tmp_path)
    dims, batch, steps, lr = [784, 100, 100, 10], 32, 12, 0.01
    weights = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(0, dims)]
    X, T = synth.mnist_like(0, 0, batch * steps)
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(struct.pack("<3q", len(dims) - 1, batch, steps))
        f.write(struct.pack(f"<{len(dims)}q", *dims))
        f.write(struct.pack("<d", lr))
        for w, b in weights:
            f.write(w.tobytes())
            f.write(b.tobytes())
        f.write(X.tobytes())
        f.write(T.tobytes())
    r = subprocess.run([exe, str(inp), str(out)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout + r.stderr
    got = np.fromfile(out, dtype=np.float64)
    losses, accs, _ = oc.mlp_train(dims, weights, X, T, batch, steps, lr)
    per_step = got[:2 * steps].reshape(steps, 2)
    assert rel_err(per_step[:, 0], losses) < REL_TOL
    assert np.array_equal(per_step[:, 1], accs)
    o = 2 * steps
    for w, b in weights:
        assert rel_err(got[o:o + w.size].reshape(w.shape), w) < REL_TOL
        o += w.size
        assert rel_err(got[o:o + b.size].reshape(b.shape), b) < REL_TOL
        o += b.size
    assert o == got.size
