"""TEST INFRASTRUCTURE: ctypes access to oracle/_build/librstorch_oracle.so.

Builds the library with `make -C oracle` when it is missing or older than its
sources (g++ only; no GPU, no reference checkout needed).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "librstorch_oracle.so")
_SOURCES = ["rstorch_oracle.cpp", "oracle_gemm.cpp", "Makefile"]

_lib = None
I64 = C.c_int64
PD = C.POINTER(C.c_double)


def build(force: bool = False) -> str:
    srcs = [os.path.join(HERE, s) for s in _SOURCES]
    stale = force or not os.path.exists(LIB) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in srcs)
    if stale:
        r = subprocess.run(["make", "-C", HERE] + (["-B"] if force else []), capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"building the oracle failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        lib = C.CDLL(LIB)
        lib.orc_xent_forward.restype = C.c_double
        lib.orc_accuracy.restype = C.c_double
        lib.orc_softmax.restype = I64
        lib.orc_max_threads.restype = C.c_int
        lib.orc_synth_uniform.restype = None
        lib.orc_synth_normal.restype = None
        _lib = lib
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(PD)


def _f64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float64)


def set_threads(n: int) -> None:
    load().orc_set_threads(C.c_int(int(n)))


def max_threads() -> int:
    return int(load().orc_max_threads())


def linear_forward(X, W, b=None, precise: bool = False) -> np.ndarray:
    X, W = _f64(X), _f64(W)
    B, cin = X.shape
    out = W.shape[0]
    assert W.shape[1] == cin
    Y = np.empty((B, out))
    bb = _f64(b).reshape(-1) if b is not None else None
    load().orc_linear_forward(_p(X), _p(W), _p(bb) if bb is not None else None, I64(B), I64(cin), I64(out),
                              _p(Y), C.c_int(int(precise)))
    return Y


def linear_backward(dY, X, W, want_db: bool = True, want_dx: bool = True, precise: bool = False):
    dY, X, W = _f64(dY), _f64(X), _f64(W)
    B, cin = X.shape
    out = W.shape[0]
    dW = np.empty((out, cin))
    db = np.empty((1, out)) if want_db else None
    dX = np.empty((B, cin)) if want_dx else None
    load().orc_linear_backward(_p(dY), _p(X), _p(W), I64(B), I64(cin), I64(out), _p(dW),
                               _p(db) if want_db else None, _p(dX) if want_dx else None,
                               C.c_int(int(precise)))
    return dW, db, dX


def relu_forward(x) -> np.ndarray:
    x = _f64(x)
    y = np.empty_like(x)
    load().orc_relu_forward(_p(x), I64(x.size), _p(y))
    return y


def relu_backward(dy, xpre) -> np.ndarray:
    dy, xpre = _f64(dy), _f64(xpre)
    dx = np.empty_like(dy)
    load().orc_relu_backward(_p(dy), _p(xpre), I64(dy.size), _p(dx))
    return dx


def softmax(x) -> tuple[np.ndarray, int]:
    x = _f64(x)
    p = np.empty_like(x)
    nan_rows = load().orc_softmax(_p(x), I64(x.shape[0]), I64(x.shape[1]), _p(p))
    return p, int(nan_rows)


def xent_forward(pred, truth) -> tuple[float, np.ndarray, int]:
    pred, truth = _f64(pred), _f64(truth)
    p = np.empty_like(pred)
    nan_rows = I64(0)
    loss = load().orc_xent_forward(_p(pred), _p(truth), I64(pred.shape[0]), I64(pred.shape[1]), _p(p),
                                   C.byref(nan_rows))
    return float(loss), p, int(nan_rows.value)


def xent_backward(p, truth) -> np.ndarray:
    p, truth = _f64(p), _f64(truth)
    g = np.empty_like(p)
    load().orc_xent_backward(_p(p), _p(truth), I64(p.size), _p(g))
    return g


def sgd_step(p, g, lr: float) -> np.ndarray:
    """Returns the updated copy of p."""
    out = _f64(p).copy()
    g = _f64(g)
    load().orc_sgd_step(_p(out), _p(g), I64(out.size), C.c_double(lr))
    return out


def argmax(x) -> np.ndarray:
    x = _f64(x)
    idx = np.empty(x.shape[0], dtype=np.int64)
    load().orc_argmax(_p(x), I64(x.shape[0]), I64(x.shape[1]), idx.ctypes.data_as(C.POINTER(I64)))
    return idx


def accuracy(pred, truth) -> float:
    pred, truth = _f64(pred), _f64(truth)
    return float(load().orc_accuracy(_p(pred), _p(truth), I64(pred.shape[0]), I64(pred.shape[1])))


def mlp_train(dims, weights, X, T, batch: int, steps: int, lr: float, skip_first_dx: bool = False,
              want_grads: bool = True):
    """Runs `steps` training steps in C++; `weights` is a list of (W, b) updated in
    place (arrays must be C-contiguous f64).  Returns (losses, accs, grads) where
    grads is the list [(dW, db), ...] of the last step."""
    L = len(dims) - 1
    X, T = _f64(X), _f64(T)
    assert X.shape[0] >= batch * steps and T.shape[0] >= batch * steps
    d = (I64 * (L + 1))(*dims)
    Wp = (PD * L)(*[_p(w) for w, _ in weights])
    bp = (PD * L)(*[_p(b) for _, b in weights])
    for w, b in weights:
        assert w.flags.c_contiguous and b.flags.c_contiguous and w.dtype == np.float64
    losses, accs = np.empty(steps), np.empty(steps)
    nparams = sum(dims[l] * dims[l + 1] + dims[l + 1] for l in range(L))
    flat = np.empty(nparams) if want_grads else None
    load().orc_mlp_train(C.c_int(L), d, Wp, bp, _p(X), _p(T), I64(batch), I64(steps), C.c_double(lr),
                         C.c_int(int(skip_first_dx)), _p(losses), _p(accs), _p(flat) if want_grads else None)
    grads = None
    if want_grads:
        grads, o = [], 0
        for l in range(L):
            nw, nb = dims[l] * dims[l + 1], dims[l + 1]
            grads.append((flat[o:o + nw].reshape(dims[l + 1], dims[l]).copy(),
                          flat[o + nw:o + nw + nb].reshape(1, nb).copy()))
            o += nw + nb
    return losses, accs, grads
