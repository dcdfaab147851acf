"""`one_hot`, `argmax`, `accuracy` (src/utils.rs:38-65)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .core import Tensor


def one_hot(x: int, n: int) -> np.ndarray:
    """Length-n f64 vector with a single 1.0 at index x (utils.rs:38-42); an index
    outside [0, n) raises like the reference's out-of-bounds panic."""
    if not 0 <= int(x) < n:
        raise IndexError(f"index {x} out of bounds for one_hot of size {n}")
    out = np.zeros(n, dtype=np.float64)
    out[int(x)] = 1.0
    return out


def argmax(arr: Tensor) -> np.ndarray:
    """Index of the maximum of every row, first maximum wins (utils.rs:44-53)."""
    ctx = arr.ctx
    out = np.empty(arr.rows, dtype=np.int64)
    ctx._check(ctx._lib.rst_argmax(ctx.handle, arr.handle, out.ctypes.data_as(C.POINTER(C.c_int64))))
    return out


def accuracy(pred: Tensor, truth: Tensor) -> float:
    """Fraction of rows whose argmax agrees (utils.rs:55-65)."""
    ctx = pred.ctx
    v = C.c_double()
    ctx._check(ctx._lib.rst_accuracy(ctx.handle, pred.handle, truth.handle, C.byref(v)))
    return v.value
