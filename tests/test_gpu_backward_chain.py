"""`rst_linear_backward_chain` against n calls of `rst_linear_backward` and against the
CPU restatement, over shapes that take the grouped launch and shapes that do not."""
import ctypes as C

import numpy as np
import pytest

import rstorch_b200 as rt
from conftest import REL_TOL, rel_err
from rstorch_b200 import _lib

pytestmark = pytest.mark.gpu


def _chain_inputs(rng, B, widths):
    """Cached inputs of a Linear/ReLU chain: X[0] random, X[l>0] post-ReLU of layer l-1."""
    ws = [rng.normal(size=(widths[l + 1], widths[l])) / np.sqrt(widths[l]) for l in range(len(widths) - 1)]
    xs = [rng.normal(size=(B, widths[0]))]
    for w in ws[:-1]:
        xs.append(np.maximum(xs[-1] @ w.T, 0.0))
    dy = rng.normal(size=(B, widths[-1]))
    return ws, xs, dy


def _numpy_backward(ws, xs, dy):
    n, B = len(ws), dy.shape[0]
    g, dws, dbs, dxs = dy, [None] * n, [None] * n, [None] * n
    for l in range(n - 1, -1, -1):
        dws[l] = g.T @ xs[l] / B
        dbs[l] = g.sum(axis=0, keepdims=True) / B
        dx = g @ ws[l]
        if l > 0:
            dx = dx * (xs[l] > 0)
        dxs[l] = dx
        g = dx
    return dws, dbs, dxs


def _handles(tensors):
    return (C.c_void_p * len(tensors))(*[t.handle.value if t is not None else None for t in tensors])


def _run_chain(ctx, ws, xs, dy, skip_first_dx):
    n = len(ws)
    tw, tx, tdy = [ctx.tensor(w) for w in ws], [ctx.tensor(x) for x in xs], ctx.tensor(dy)
    dw = [ctx.empty(*w.shape) for w in ws]
    db = [ctx.empty(1, w.shape[0]) for w in ws]
    dx = [None if (l == 0 and skip_first_dx) else ctx.empty(*xs[l].shape) for l in range(n)]
    masks = (C.c_ubyte * n)(*[0] + [1] * (n - 1))
    before = ctx.launch_count()
    ctx._check(ctx._lib.rst_linear_backward_chain(ctx.handle, n, tdy.handle, _handles(tx), _handles(tw), masks,
                                                  _handles(dw), _handles(db), _handles(dx)))
    launches = ctx.launch_count() - before
    return ([t.numpy() for t in dw], [t.numpy() for t in db],
            [t.numpy() if t is not None else None for t in dx], launches)


@pytest.mark.parametrize("B,widths,skip", [
    (32, [784, 100, 100, 10], True),        # batch-32 README model: grouped
    (4096, [784, 100, 100, 10], True),      # batch-4096: grouped with split K
    (256, [64, 48, 32, 16, 8], False),      # four layers, dX of the input wanted
    (64, [20, 30], False),                  # a single layer: nothing to group
    (128, [36, 50, 24, 12, 40, 8], True),   # five layers: one group of four and a single
    (50, [33, 20, 7], False),               # odd widths: plain-load kernels, no grouping
])
def test_chain_matches_layer_by_layer_and_numpy(ctx, B, widths, skip):
    rng = np.random.default_rng(B + len(widths))
    ws, xs, dy = _chain_inputs(rng, B, widths)
    n = len(ws)
    dw_c, db_c, dx_c, launches = _run_chain(ctx, ws, xs, dy, skip)

    # layer by layer through rst_linear_backward
    g = ctx.tensor(dy)
    for l in range(n - 1, -1, -1):
        x, w = ctx.tensor(xs[l]), ctx.tensor(ws[l])
        dw, db = ctx.empty(*ws[l].shape), ctx.empty(1, ws[l].shape[0])
        want_dx = not (l == 0 and skip)
        dx = ctx.empty(*xs[l].shape) if want_dx else None
        ctx._check(ctx._lib.rst_linear_backward(ctx.handle, g.handle, x.handle, w.handle,
                                                x.handle if (l > 0 and want_dx) else None,
                                                dw.handle, db.handle, dx.handle if dx is not None else None))
        assert rel_err(dw_c[l], dw.numpy()) < 1e-13
        assert rel_err(db_c[l], db.numpy()) < 1e-13
        if want_dx:
            assert np.array_equal(dx_c[l], dx.numpy())      # same kernel, same launch shape
        g = dx

    dw_n, db_n, dx_n = _numpy_backward(ws, xs, dy)
    for l in range(n):
        assert rel_err(dw_c[l], dw_n[l]) < REL_TOL
        assert rel_err(db_c[l], db_n[l]) < REL_TOL
        if dx_c[l] is not None:
            assert rel_err(dx_c[l], dx_n[l]) < REL_TOL
    assert (dx_c[0] is None) == skip

    if widths == [784, 100, 100, 10]:
        # two dX products, one grouped dW launch, at most one grouped reduce
        assert launches <= 4


def test_chain_is_deterministic_run_to_run(ctx):
    rng = np.random.default_rng(5)
    ws, xs, dy = _chain_inputs(rng, 4096, [784, 100, 100, 10])
    a = _run_chain(ctx, ws, xs, dy, True)
    b = _run_chain(ctx, ws, xs, dy, True)
    for l in range(3):
        assert np.array_equal(a[0][l], b[0][l]) and np.array_equal(a[1][l], b[1][l])


def test_chain_argument_errors(ctx):
    rng = np.random.default_rng(6)
    ws, xs, dy = _chain_inputs(rng, 16, [8, 6, 4])
    tw, tx, tdy = [ctx.tensor(w) for w in ws], [ctx.tensor(x) for x in xs], ctx.tensor(dy)
    dw = [ctx.empty(*w.shape) for w in ws]
    db = [ctx.empty(1, w.shape[0]) for w in ws]
    dx = [ctx.empty(*x.shape) for x in xs]
    lib = ctx._lib
    # an inner dX is needed by the layer in front of it
    status = lib.rst_linear_backward_chain(ctx.handle, 2, tdy.handle, _handles(tx), _handles(tw), None,
                                           _handles(dw), _handles(db), _handles([dx[0], None]))
    assert status == _lib.RST_ERR_INVALID_ARG
    # a weight of the wrong shape is a shape error, as in the single-layer call
    status = lib.rst_linear_backward_chain(ctx.handle, 2, tdy.handle, _handles(tx), _handles([tw[1], tw[0]]), None,
                                           _handles(dw), _handles(db), _handles(dx))
    assert status == _lib.RST_ERR_SHAPE
    assert lib.rst_linear_backward_chain(ctx.handle, 0, tdy.handle, _handles(tx), _handles(tw), None,
                                         _handles(dw), _handles(db), _handles(dx)) == _lib.RST_ERR_INVALID_ARG


def test_sequential_backward_uses_the_chain_and_matches_unfused_layers(ctx):
    """`Sequential.backward` of a small MLP (one library call) against the same layers
    called one by one."""
    def build():
        return [rt.Linear(20, 16, rt.KaimingNormal(3)), rt.ReLU(), rt.Linear(16, 12, rt.KaimingNormal(4)),
                rt.ReLU(), rt.Linear(12, 6, rt.KaimingNormal(5))]
    rng = np.random.default_rng(8)
    x, g = rng.normal(size=(40, 20)), rng.normal(size=(40, 6))
    seq = rt.Sequential([rt.Identity()] + build())
    assert seq._small_linear_chain() is not None
    y = seq.forward(ctx.tensor(x))
    dx = seq.backward(ctx.tensor(g))
    layers = build()
    h = ctx.tensor(x)
    for layer in layers:
        h = layer.forward(h)
    d = ctx.tensor(g)
    for layer in reversed(layers):
        d = layer.backward(d)
    assert rel_err(y.numpy(), h.numpy()) < 1e-13
    assert rel_err(dx.numpy(), d.numpy()) < 1e-13
    for p, q in zip(seq.parameters(), [p for layer in layers for p in layer.parameters()]):
        assert rel_err(p.grad.numpy(), q.grad.numpy()) < 1e-12
