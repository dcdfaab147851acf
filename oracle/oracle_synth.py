"""TEST INFRASTRUCTURE: the benchmark's seeded input streams, restated over the CPU
oracle's own generator (oracle/rstorch_oracle.cpp: orc_synth_uniform / orc_synth_normal).

The CPU arm of the benchmark draws its weights and batches from here, so that it loads
nothing of the library it is timed against; tests/test_oracle.py holds every function
below to the library's generator bit for bit.  Streams: word i of stream `key` is
splitmix64(key + (i+1)·φ64); keys come from blake2b("seed:purpose:index").
"""
from __future__ import annotations

import ctypes as C
import hashlib

import numpy as np

from . import oracle_c

U64 = C.c_uint64


def stream_key(seed: int, purpose: str, index: int = 0) -> int:
    h = hashlib.blake2b(f"{seed}:{purpose}:{index}".encode(), digest_size=8).digest()
    return int.from_bytes(h, "little")


def uniform(key: int, n: int, offset: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float64)
    oracle_c.load().orc_synth_uniform(U64(key), U64(n), U64(offset), out.ctypes.data_as(oracle_c.PD))
    return out


def normal(key: int, n: int, std: float = 1.0, mean: float = 0.0, offset: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float64)
    oracle_c.load().orc_synth_normal(U64(key), U64(n), U64(offset), C.c_double(mean), C.c_double(std),
                                     out.ctypes.data_as(oracle_c.PD))
    return out


def integers(key: int, n: int, high: int, offset: int = 0) -> np.ndarray:
    return (uniform(key, n, offset) * high).astype(np.int64)


def one_hot(labels: np.ndarray, classes: int) -> np.ndarray:
    out = np.zeros((labels.shape[0], classes), dtype=np.float64)
    out[np.arange(labels.shape[0]), labels] = 1.0
    return out


def mnist_like(seed: int, first_sample: int, n: int, features: int = 784, classes: int = 10,
               zero_fraction: float = 0.81):
    """MNIST-shaped stream: `zero_fraction` exact zeros, the rest in (0, 1]; one-hot labels."""
    off = first_sample * features
    keep = uniform(stream_key(seed, "mnist_like.zero"), n * features, off) >= zero_fraction
    vals = 1.0 - uniform(stream_key(seed, "mnist_like.value"), n * features, off)
    x = np.where(keep, vals, 0.0).reshape(n, features)
    labels = integers(stream_key(seed, "mnist_like.label"), n, classes, first_sample)
    return x, one_hot(labels, classes)


def gaussian_batch(seed: int, step: int, first_row: int, rows: int, features: int, classes: int, global_batch: int):
    """Rows [first_row, first_row + rows) of the step's global batch: X ~ N(0,1), uniform one-hot labels."""
    row0 = step * global_batch + first_row
    x = normal(stream_key(seed, "gaussian.x"), rows * features, offset=row0 * features).reshape(rows, features)
    labels = integers(stream_key(seed, "gaussian.label"), rows, classes, row0)
    return x, one_hot(labels, classes)


def mlp_weights(seed: int, dims: list[int]):
    """Per Linear: W (out, in) ~ N(0, 1/sqrt(in)) from stream ("weight", layer), b = 0
    (src/module/init/he.rs:9-15, init/mod.rs:15-17)."""
    out = []
    for layer in range(len(dims) - 1):
        fan_in, fan_out = dims[layer], dims[layer + 1]
        w = normal(stream_key(seed, "weight", layer), fan_in * fan_out, std=1.0 / np.sqrt(fan_in))
        out.append((w.reshape(fan_out, fan_in), np.zeros((1, fan_out), dtype=np.float64)))
    return out
