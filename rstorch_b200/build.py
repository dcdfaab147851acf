"""Builds librstorch_b200.so in-tree with nvcc for sm_100a.

    python -m rstorch_b200.build [--force] [--define NAME ...]

Object files go to rstorch_b200/csrc/build/, the library next to this file.  nvcc
cross-compiles without a GPU, so this runs on any host that has CUDA 12.9+.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "librstorch_b200.so")
SOURCES = ["runtime.cu", "ops.cu", "gemm_f64.cu", "xent.cu", "sgd.cu", "elementwise.cu",
           "stager.cu", "comm.cu", "probe.cu", "synth.cu", "dataset.cu"]
HEADERS = ["common.h", "mma_f64.cuh", os.path.join("..", "..", "include", "rstorch_b200.h")]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; librstorch_b200.so cannot be built")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build_library(force: bool = False, defines: tuple[str, ...] = (), verbose: bool = False) -> str:
    """Compiles every .cu of the package and links the shared library; returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    flags = ARCH + ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
                    "-Xptxas", "-v" if verbose else "-warn-spills"]
    flags += [f"-D{d}" for d in defines]
    stamp = os.path.join(OBJ, "flags.txt")
    flag_text = " ".join(flags)
    if not os.path.exists(stamp) or open(stamp).read() != flag_text:
        force = True

    def compile_one(src: str) -> tuple[str, str]:
        obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
        path = os.path.join(CSRC, src)
        if force or _stale(obj, [path] + headers):
            r = subprocess.run([nvcc] + flags + ["-c", path, "-o", obj], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
            return obj, r.stderr
        return obj, ""

    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(compile_one, sources))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    if force or _stale(LIB, objs):
        r = subprocess.run([nvcc] + ARCH + ["-shared", "-o", LIB] + objs + ["-ldl"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(flag_text)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[])
    a = ap.parse_args()
    print(build_library(a.force, tuple(a.define), a.verbose))
