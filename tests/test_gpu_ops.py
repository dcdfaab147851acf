"""Parity of every kernel, called through the C ABI, with the CPU restatement."""
import ctypes as C

import numpy as np
import pytest

import rstorch_b200 as rt
from conftest import REL_TOL, rel_err
from rstorch_b200 import _lib

pytestmark = pytest.mark.gpu


def A(x):
    return np.array(x, dtype=np.float64)


class Fixed(rt.InitParameters):
    def __init__(self, w, b):
        self.w, self.b = A(w), A(b)

    def weight(self, i, o):
        return self.w

    def bias(self, i, o):
        return self.b


# ---- the reference's own unit tests, through the device path -------------------------
def test_kat_linear_forward(ctx, kat):
    k = kat["linear_forward"]
    m = rt.Linear.new_with_kernel(2, 1, Fixed(k["weight"], k["bias"]))
    y = m.forward(ctx.tensor(A(k["input"]))).numpy()
    assert np.max(np.abs(y - A(k["expected"]))) <= kat["tolerance"]


def test_kat_linear_backward(ctx, kat):
    k = kat["linear_backward"]
    m = rt.Linear.new_with_kernel(2, 1, Fixed(k["weight"], k["bias"]))
    m.forward(ctx.tensor(A(k["input"])))
    dx = m.backward(ctx.tensor(A(k["gradient"]))).numpy()
    assert m.grad_weight.shape == m.weight.shape and m.grad_bias.shape == m.bias.shape
    tol = kat["tolerance"]
    assert np.max(np.abs(m.grad_weight.numpy() - A(k["expected_grad_weight"]))) <= tol
    assert np.max(np.abs(m.grad_bias.numpy() - A(k["expected_grad_bias"]))) <= tol
    assert np.max(np.abs(dx - A(k["expected_grad_input"]))) <= tol


def test_kat_relu_identity(ctx, kat):
    f, b, i = kat["relu_forward"], kat["relu_backward"], kat["identity"]
    m = rt.ReLU()
    assert np.array_equal(m.forward(ctx.tensor(A(f["input"]))).numpy(), A(f["expected"]))
    m.forward(ctx.tensor(A(b["input"])))
    assert np.array_equal(m.backward(ctx.tensor(A(b["gradient"]))).numpy(), A(b["expected"]))
    ident = rt.Identity()
    x = ctx.tensor(A(i["input"]))
    assert np.array_equal(ident.forward(x).numpy(), A(i["expected"]))
    assert np.array_equal(ident.backward(x).numpy(), A(i["expected"]))


def test_kat_softmax_rows(ctx, kat):
    k = kat["softmax_rows_sum_to_one"]
    x = ctx.tensor(A(k["input"]))
    p = ctx.empty(3, 2)
    ctx._check(ctx._lib.rst_softmax(ctx.handle, x.handle, p.handle))
    p = p.numpy()
    assert np.max(np.abs(p.sum(axis=1) - 1.0)) <= kat["tolerance"]
    assert abs(p.sum() - 3.0) <= 4 * np.finfo(float).eps


def test_kat_sgd_zero_gradient(ctx, kat):
    lin = rt.Linear(2, 2, ctx=ctx)
    w0 = lin.weight.numpy()
    lin.forward(ctx.zeros(2, 2))
    lin.backward(ctx.zeros(2, 2))
    rt.SGD.new(kat["sgd_zero_gradient"]["lr"]).step(lin)
    assert np.array_equal(lin.weight.numpy(), w0)


# ---- Linear: all three GEMM layouts, every dispatch path -------------------------------
LINEAR_SHAPES = [
    (1, 2, 2),          # smallest TMA-addressable shape
    (3, 5, 7),          # odd pitches: plain-load kernel
    (32, 784, 100),     # C1 layer 1 (split-K forward)
    (32, 100, 10),      # C1 head
    (64, 100, 100),
    (20, 70, 44),       # 32x32 tiles, ragged rows and columns
    (200, 24, 18),      # 32x32 tiles in dW (18 rows) and dX (24 columns), 64x64 nowhere
    (500, 2000, 16),    # 32x32 tiles with split K: forward (16 columns) and dW + db (16 rows)
    (257, 130, 66),     # ragged in every dimension, 64x64 tiles
    (4096, 784, 100),   # C2 layer 1 (split-K dW)
    (2048, 1024, 2048), # 128x128 tiles, >= 148 of them
    (2048, 2048, 2048), # 256 large tiles = 1.73 waves: split K four ways in all three products
    (1920, 272, 1288),  # 128x128 tiles with ragged edges in M, N and K
    (3000, 4000, 4100), # 792 / 768 / 1056 large tiles, ragged everywhere, 188-257 k-tiles: the last, partly
                        # filled wave of all three products is handed out in k runs (tail launch + fix-up)
]


@pytest.mark.parametrize("B,cin,cout", LINEAR_SHAPES)
def test_linear_forward_backward_parity(ctx, oc, B, cin, cout):
    rng = np.random.default_rng(B + 7 * cin + 13 * cout)
    X = rng.standard_normal((B, cin))
    X[X < -0.5] = 0.0                                  # exact zeros as a ReLU output has
    W, b = rng.standard_normal((cout, cin)) / np.sqrt(cin), rng.standard_normal((1, cout))
    dY = rng.standard_normal((B, cout))
    lin = rt.Linear.new_with_kernel(cin, cout, Fixed(W, b))
    xd = ctx.tensor(X)

    y = lin.forward(xd).numpy()
    assert rel_err(y, oc.linear_forward(X, W, b)) < REL_TOL
    dx = lin.backward(ctx.tensor(dY)).numpy()
    dW, db, dX = oc.linear_backward(dY, X, W)
    assert rel_err(lin.grad_weight.numpy(), dW) < REL_TOL
    assert rel_err(lin.grad_bias.numpy(), db) < REL_TOL
    assert rel_err(dx, dX) < REL_TOL

    # fused epilogues: ReLU in forward, ReLU mask (from the cached input) in dX, dX skipped
    y_relu = lin._forward(xd, fuse_relu=True).numpy()
    assert np.array_equal(y_relu, np.maximum(y, 0.0))
    dx_masked = lin._backward(ctx.tensor(dY), relu_mask=True, need_input_grad=True).numpy()
    assert np.array_equal(dx_masked, dx * (X > 0.0))
    lin._forward(xd, fuse_relu=False)
    assert lin._backward(ctx.tensor(dY), relu_mask=False, need_input_grad=False) is None
    assert rel_err(lin.grad_weight.numpy(), dW) < REL_TOL
    ctx.check_device()


@pytest.mark.parametrize("B,cin,cout", [(3, 5, 7), (32, 100, 10), (257, 130, 66), (2048, 1024, 2048)])
def test_linear_without_bias_parity(ctx, oc, B, cin, cout):
    """`bias: None` (linear.rs:51-53, 65-67, 74-77): b = NULL forward, db = NULL backward,
    the ReLU that cannot ride in a bias-less epilogue, and the one-pair parameter list."""
    rng = np.random.default_rng(B + cin + cout)
    X, W = rng.standard_normal((B, cin)), rng.standard_normal((cout, cin)) / np.sqrt(cin)
    X[X < -0.5] = 0.0
    dY = rng.standard_normal((B, cout))
    lin = rt.Linear.without_bias(cin, cout, Fixed(W, np.zeros((1, cout))))
    xd = ctx.tensor(X)
    y = lin.forward(xd).numpy()
    assert rel_err(y, oc.linear_forward(X, W, None)) < REL_TOL
    dx = lin.backward(ctx.tensor(dY)).numpy()
    dW, _, dX = oc.linear_backward(dY, X, W, want_db=False)
    assert rel_err(lin.grad_weight.numpy(), dW) < REL_TOL and rel_err(dx, dX) < REL_TOL
    assert lin.grad_bias is None and lin.bias is None
    params = lin.parameters()
    assert len(params) == 1 and params[0].parm is lin.weight
    # fused call sites: ReLU after a bias-less product, mask in dX
    y_relu = lin._forward(xd, fuse_relu=True).numpy()
    assert np.array_equal(y_relu, np.maximum(y, 0.0))
    dx_masked = lin._backward(ctx.tensor(dY), relu_mask=True, need_input_grad=True).numpy()
    assert np.array_equal(dx_masked, dx * (X > 0.0))
    # inside a container, next to layers that do have a bias; SGD moves the one tensor it is given
    seq = rt.sequential(rt.Linear.new_with_kernel(cin, cout, Fixed(W, np.ones((1, cout)))), rt.ReLU(),
                        rt.Linear.without_bias(cout, 4, Fixed(np.ones((4, cout)), np.zeros((1, 4)))))
    out = seq.forward(xd)
    seq.backward(ctx.tensor(np.ones((B, 4))))
    assert out.shape == (B, 4) and len(seq.parameters()) == 3
    before = seq.layers[2].weight.numpy()
    rt.SGD.new(0.5).step(seq)
    assert np.array_equal(seq.layers[2].weight.numpy(), oc.sgd_step(before, seq.layers[2].grad_weight.numpy(), 0.5))
    ctx.check_device()


def test_bounded_wait_runs_out_and_the_context_stays_usable(ctx, oc):
    """A kernel whose producer never copies a tile: every consumer wait runs out after the
    given limit, the kernel reports it through the status word and returns; the next check
    returns RST_ERR_DEVICE_TIMEOUT, clears the word, and ordinary launches pass parity."""
    ctx.check_device()
    ctx._check(ctx._lib.rst_selftest_wait_expiry(ctx.handle, 100_000))
    with pytest.raises(rt.RstError) as e:
        ctx.check_device()
    assert e.value.status == _lib.RST_ERR_DEVICE_TIMEOUT and "bounded wait" in str(e.value)
    ctx.check_device()                                     # cleared
    rng = np.random.default_rng(5)
    X, W, b = rng.standard_normal((64, 64)), rng.standard_normal((64, 64)), rng.standard_normal((1, 64))
    lin = rt.Linear.new_with_kernel(64, 64, Fixed(W, b))
    assert rel_err(lin.forward(ctx.tensor(X)).numpy(), oc.linear_forward(X, W, b)) < REL_TOL
    ctx.check_device()
    assert ctx._lib.rst_selftest_wait_expiry(ctx.handle, 0) == _lib.RST_ERR_INVALID_ARG
    assert ctx._lib.rst_selftest_wait_expiry(ctx.handle, 10**9) == _lib.RST_ERR_INVALID_ARG


def test_tensor_checksum_tells_bit_patterns_apart(ctx):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((300, 77))
    t1, t2 = ctx.tensor(a), ctx.tensor(a)
    assert t1.checksum() == t2.checksum() == t1.checksum()
    b = a.copy(); b[17, 3] = np.nextafter(b[17, 3], np.inf)         # one ulp
    assert ctx.tensor(b).checksum() != t1.checksum()
    c = a.copy(); c[0, 0], c[0, 1] = a[0, 1], a[0, 0]                # same values, other order
    assert ctx.tensor(c).checksum() != t1.checksum()
    z = np.zeros((4, 4)); nz = z.copy(); nz[1, 1] = -0.0
    assert ctx.tensor(z).checksum() != ctx.tensor(nz).checksum()    # bits, not values
    assert ctx.empty(0, 5).checksum() == 0


def test_tail_launch_is_taken_and_agrees_with_whole_tiles(ctx, monkeypatch):
    """3000 x 4100 x 4000 forward = 792 tiles of 128 x 128 = 5.35 waves on 148 SMs: the product
    runs as main launch + tail launch + fix-up, and gives the sums of the whole-tile path in
    another order (a context created with RSTORCH_B200_STREAM_TAIL=0 takes that path)."""
    rng = np.random.default_rng(11)
    X, W, b = rng.standard_normal((3000, 4000)), rng.standard_normal((4100, 4000)) / 64.0, rng.standard_normal((1, 4100))
    lin = rt.Linear.new_with_kernel(4000, 4100, Fixed(W, b))
    xd = ctx.tensor(X)
    before = ctx.launch_count()
    y = lin._forward(xd, fuse_relu=True).numpy()
    sms = 148
    expected = 3 if (792 % sms) and ((sms - 792 % sms) * 250 // sms >= 100) else 1
    assert ctx.launch_count() - before == expected
    monkeypatch.setenv("RSTORCH_B200_STREAM_TAIL", "0")
    plain = rt.Context(0)
    try:
        lin2 = rt.Linear.new_with_kernel(4000, 4100, Fixed(W, b))
        before = plain.launch_count()
        y2 = lin2._forward(plain.tensor(X), fuse_relu=True).numpy()
        assert plain.launch_count() - before == 1
    finally:
        plain.close()
    assert rel_err(y, y2) < 1e-13 and np.array_equal(y == 0.0, y2 == 0.0)
    ctx.check_device()


def test_linear_is_deterministic_run_to_run(ctx):
    rng = np.random.default_rng(0)
    X, W, b = rng.standard_normal((512, 300)), rng.standard_normal((200, 300)), rng.standard_normal((1, 200))
    lin = rt.Linear.new_with_kernel(300, 200, Fixed(W, b))
    xd, gd = ctx.tensor(X), ctx.tensor(rng.standard_normal((512, 200)))
    outs = []
    for _ in range(3):
        y = lin.forward(xd).numpy()
        dx = lin.backward(gd).numpy()
        outs.append((y, dx, lin.grad_weight.numpy(), lin.grad_bias.numpy()))
    for o in outs[1:]:
        for a, b_ in zip(o, outs[0]):
            assert np.array_equal(a, b_)


@pytest.mark.parametrize("B,cin,cout", [(4096, 784, 100), (1024, 512, 256), (2048, 1024, 2048)])
def test_stage_ring_reuse_is_race_free(ctx, B, cin, cout):
    """Shapes whose k loop wraps the shared-memory stage ring several times, with
    several CTAs resident per SM (split-K): thirty back-to-back repeats must be
    bit-identical and correct.  Guards the ordering between the consumers' shared
    loads and the TMA refill of a stage."""
    rng = np.random.default_rng(1)
    X, W = rng.standard_normal((B, cin)), rng.standard_normal((cout, cin))
    dY = rng.standard_normal((B, cout))
    lin = rt.Linear.new_with_kernel(cin, cout, Fixed(W, np.zeros((1, cout))))
    xd, gd = ctx.tensor(X), ctx.tensor(dY)
    first = None
    for _ in range(30):
        y = lin._forward(xd, False)
        dx = lin._backward(gd, False, True)
        cur = (y.numpy(), lin.grad_weight.numpy(), dx.numpy())
        if first is None:
            first = cur
            assert rel_err(cur[0], X @ W.T) < REL_TOL
            assert rel_err(cur[1], dY.T @ X / B) < REL_TOL
            assert rel_err(cur[2], dY @ W) < REL_TOL
        else:
            for a, b in zip(cur, first):
                assert np.array_equal(a, b)


def test_linear_shape_errors(ctx):
    lin = rt.Linear(4, 3, ctx=ctx)
    with pytest.raises(rt.RstError) as e:
        lin.forward(ctx.zeros(2, 5))
    assert e.value.status == _lib.RST_ERR_SHAPE
    lin.forward(ctx.zeros(2, 4))
    with pytest.raises(rt.RstError) as e:
        lin.backward(ctx.zeros(2, 4))
    assert e.value.status == _lib.RST_ERR_SHAPE
    other = rt.Context(0)
    try:
        mine, theirs = ctx.zeros(2, 4), other.zeros(2, 4)
        st = ctx._lib.rst_relu_forward(ctx.handle, theirs.handle, mine.handle)
        assert st == _lib.RST_ERR_FOREIGN_HANDLE
        theirs.free()
    finally:
        other.close()


# ---- ReLU ------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(1, 1), (3, 7), (129, 1001), (4096, 100)])
def test_relu_parity(ctx, oc, shape):
    rng = np.random.default_rng(shape[0])
    x = rng.standard_normal(shape)
    x.flat[::7] = 0.0
    x.flat[3::11] = -0.0
    if x.size > 5:
        x.flat[5] = np.nan
    g = rng.standard_normal(shape)
    m = rt.ReLU()
    assert np.array_equal(m.forward(ctx.tensor(x)).numpy(), oc.relu_forward(x))
    assert np.array_equal(m.backward(ctx.tensor(g)).numpy(), oc.relu_backward(g, x), equal_nan=True)


# ---- softmax / cross-entropy / accuracy ---------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(1, 1), (5, 2), (32, 10), (4096, 10), (33, 17), (100, 32), (64, 100),
                                       (31, 500), (256, 1000), (8, 1024), (5, 1500), (3000, 1000), (40, 2048),
                                       (7, 2049)])
def test_xent_parity(ctx, oc, rows, cols):
    rng = np.random.default_rng(rows * 31 + cols)
    x = rng.standard_normal((rows, cols)) * 4
    t = np.eye(cols)[rng.integers(0, cols, rows)]
    # make ties and repeated maxima part of the input
    if cols > 2:
        x[0, 1] = x[0, 2] = x[0].max() + 1.0
    loss_fn = rt.CrossEntropyLoss()
    xd, td = ctx.tensor(x), ctx.tensor(t)
    loss = loss_fn.forward(xd, td)
    want_loss, p, _ = oc.xent_forward(x, t)
    assert abs(loss - want_loss) <= REL_TOL * abs(want_loss)
    assert rel_err(loss_fn.backward().numpy(), oc.xent_backward(p, t)) < REL_TOL
    assert loss_fn.last_accuracy == oc.accuracy(x, t)                 # bit-exact
    assert rt.accuracy(xd, td) == oc.accuracy(x, t)
    assert np.array_equal(rt.argmax(xd), oc.argmax(x))
    sm = ctx.empty(rows, cols)
    ctx._check(ctx._lib.rst_softmax(ctx.handle, xd.handle, sm.handle))
    assert rel_err(sm.numpy(), p) < REL_TOL


def test_xent_soft_labels_and_underflow(ctx, oc):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((16, 10))
    t = rng.random((16, 10))
    t /= t.sum(axis=1, keepdims=True)                                  # soft labels are legal
    lf = rt.CrossEntropyLoss()
    loss = lf.forward(ctx.tensor(x), ctx.tensor(t))
    want, p, _ = oc.xent_forward(x, t)
    assert abs(loss - want) <= REL_TOL * abs(want)
    # 0 * ln(0) = NaN, as in cross_entropy.rs:38
    x2, t2 = np.array([[0.0, -800.0]]), np.array([[1.0, 0.0]])
    assert np.isnan(oc.xent_forward(x2, t2)[0])
    assert np.isnan(rt.CrossEntropyLoss().forward(ctx.tensor(x2), ctx.tensor(t2)))


@pytest.mark.parametrize("cols", [10, 1000])
def test_xent_nan_logit_is_an_error_like_the_reference_panic(ctx, cols):
    x = np.zeros((4, cols))
    x[2, 3] = np.nan
    t = np.eye(cols)[[0, 1, 2, 3]]
    with pytest.raises(rt.RstError) as e:
        rt.CrossEntropyLoss().forward(ctx.tensor(x), ctx.tensor(t))
    assert e.value.status == _lib.RST_ERR_NAN


def test_xent_wide_rows_soft_labels_ties_and_nan_targets(ctx, oc):
    """The one-CTA-per-row kernel (129 to 2048 classes): soft labels, a tie across two warps'
    columns, a NaN in column 0 of the targets (argmax answers 0, as the fold does)."""
    rng = np.random.default_rng(12)
    x = rng.standard_normal((9, 700)) * 3
    t = rng.random((9, 700))
    t /= t.sum(axis=1, keepdims=True)
    x[1, 40] = x[1, 650] = x[1].max() + 2.0              # first of two equal maxima wins
    t[2, 5] = t[2, 300] = 0.9
    t[3, 0] = np.nan
    lf = rt.CrossEntropyLoss()
    xd, td = ctx.tensor(x), ctx.tensor(t)
    loss = lf.forward(xd, td)
    want, p, _ = oc.xent_forward(x, t)
    assert np.isnan(loss) and np.isnan(want)             # the NaN target poisons the whole-matrix sum
    got = lf.backward().numpy()
    ref = oc.xent_backward(p, t)
    ok = ~np.isnan(ref)
    assert np.array_equal(np.isnan(got), np.isnan(ref)) and rel_err(got[ok], ref[ok]) < REL_TOL
    assert lf.last_accuracy == oc.accuracy(x, t)
    assert np.array_equal(rt.argmax(td), oc.argmax(t)) and rt.argmax(xd)[1] == 40


def test_argmax_first_maximum_wins(ctx, oc):
    x = np.array([[1.0, 3.0, 3.0, 2.0], [5.0, 5.0, 5.0, 5.0], [np.nan, 9.0, 1.0, 0.0],
                  [1.0, np.nan, 7.0, 7.0], [-np.inf, -np.inf, np.nan, -np.inf]])
    assert rt.argmax(ctx.tensor(x)).tolist() == oc.argmax(x).tolist() == [1, 0, 0, 2, 0]
    wide = np.zeros((3, 1300))
    wide[0, 1200] = wide[0, 77] = 2.0
    wide[1, :] = -1.0
    wide[2, 0] = np.nan
    wide[2, 5] = 9.0
    assert rt.argmax(ctx.tensor(wide)).tolist() == oc.argmax(wide).tolist() == [77, 0, 0]


@pytest.mark.parametrize("cols", [10, 100, 300, 1000, 2048, 3000])
def test_xent_of_an_empty_batch_is_nan_like_the_reference(ctx, cols):
    """Zero rows: `-(Σ t·ln p) / 0` is 0/0 = NaN in the reference (cross_entropy.rs:38) for
    every class count; no launch may fail on the empty grid."""
    logits, truth = ctx.empty(0, cols), ctx.empty(0, cols)
    loss_fn = rt.CrossEntropyLoss()
    loss = loss_fn.forward(logits, truth)
    assert np.isnan(loss) and np.isnan(loss_fn.last_accuracy)
    assert loss_fn.backward().shape == (0, cols)
    ctx.check_device()


def test_result_slot_misuse(ctx):
    loss, acc = C.c_double(), C.c_double()
    st = ctx._lib.rst_xent_result(ctx.handle, 10_000, C.byref(loss), C.byref(acc))
    assert st == _lib.RST_ERR_INVALID_ARG
    fresh = rt.Context(0)
    try:
        st = fresh._lib.rst_xent_result(fresh.handle, 0, C.byref(loss), C.byref(acc))
        assert st == _lib.RST_ERR_STATE
    finally:
        fresh.close()


# ---- SGD -----------------------------------------------------------------------------------
def test_sgd_multi_tensor_is_bit_exact(ctx, oc):
    rng = np.random.default_rng(2)
    sizes = [1, 2, 3, 4095, 4096, 4097, 8192 * 3 + 5, 100 * 784, 100, 10]
    params = [rng.standard_normal((1, n)) * 0.02 for n in sizes]
    grads = [rng.standard_normal((1, n)) * 1e-3 for n in sizes]
    pd, gd = [ctx.tensor(p) for p in params], [ctx.tensor(g) for g in grads]
    from rstorch_b200.core import handle_array
    for step in range(2):
        ctx._check(ctx._lib.rst_sgd_step(ctx.handle, len(pd), handle_array(pd), handle_array(gd), 0.01))
        params = [oc.sgd_step(p, g, 0.01) for p, g in zip(params, grads)]
    for got, want in zip(pd, params):
        assert np.array_equal(got.numpy(), want)


def test_sgd_on_unaligned_slices_of_one_arena(ctx, oc):
    rng = np.random.default_rng(4)
    sizes = [5, 4099, 3, 12288, 7]
    total = sum(sizes)
    P, G = rng.standard_normal((1, total)), rng.standard_normal((1, total))
    pa, ga = ctx.tensor(P), ctx.tensor(G)
    ps, gs, o = [], [], 0
    for n in sizes:
        ps.append(pa.slice(o, 1, n)); gs.append(ga.slice(o, 1, n)); o += n
    from rstorch_b200.core import handle_array
    ctx._check(ctx._lib.rst_sgd_step(ctx.handle, len(ps), handle_array(ps), handle_array(gs), 0.5))
    assert np.array_equal(pa.numpy(), oc.sgd_step(P, G, 0.5))
    with pytest.raises(rt.RstError) as e:
        pa.slice(total - 1, 1, 2)
    assert e.value.status == _lib.RST_ERR_SHAPE


def test_sgd_shape_mismatch(ctx):
    from rstorch_b200.core import handle_array
    a, b = ctx.zeros(2, 3), ctx.zeros(3, 2)
    st = ctx._lib.rst_sgd_step(ctx.handle, 1, handle_array([a]), handle_array([b]), 0.1)
    assert st == _lib.RST_ERR_SHAPE


# ---- allocator, staging, graph replay ---------------------------------------------------------
def test_caching_allocator_reuses_blocks_and_honours_the_limit():
    c = rt.Context(0)
    try:
        t = c.empty(1000, 1000)
        s1 = c.memory_stats()
        assert s1["in_use"] >= 8_000_000 and s1["driver_allocs"] == 1
        p1 = t.data_ptr()
        t.free()
        u = c.empty(1000, 1000)
        s2 = c.memory_stats()
        assert u.data_ptr() == p1 and s2["cache_hits"] == 1 and s2["driver_allocs"] == 1
        u.free()
        c.empty_cache()
        assert c.memory_stats()["reserved"] == 0
        c.set_memory_limit(4 << 20)
        with pytest.raises(rt.RstError) as e:
            c.empty(1024, 1024)          # 8 MiB
        assert e.value.status == _lib.RST_ERR_OOM
        small = c.empty(256, 256)        # 512 KiB still fits
        assert small.numel == 65536
    finally:
        c.close()


def test_data_loader_iter_array_matches_the_reference_test(ctx, kat):
    k = kat["data_loader_iter_array"]
    n = k["samples"]
    samples = np.repeat(np.arange(n, dtype=np.float64), 16).reshape(n, 4, 4)
    targets = np.repeat(np.arange(n, dtype=np.float64), 4).reshape(n, 4)
    ds = rt.ArrayDataset(samples, targets)
    dl = rt.DataLoader(ds, k["batch_size"], False, rt.SequentialSampler(len(ds)), ctx, slots=2)
    assert len(dl) == k["expected_len"]
    batches = [(x.numpy(), t.numpy()) for x, t in dl.iter_array()]
    assert len(batches) == 3                               # the 4 left-over samples are dropped
    for i, (x, t) in enumerate(batches):
        lo = i * 32
        assert np.array_equal(x, samples[lo:lo + 32].reshape(32, 16))
        assert np.array_equal(t, targets[lo:lo + 32])
    dl1 = rt.DataLoader(ds, 32, False, rt.SequentialSampler(len(ds)), ctx, slots=1)
    assert [x.numpy()[0, 0] for x, _ in dl1.iter_array()] == [0.0, 32.0, 64.0]
    dl.close(); dl1.close()


def test_graph_replay_reproduces_the_eager_step(ctx, oc):
    from rstorch_b200 import synth
    dims = [20, 16, 12, 5]
    W = synth.mlp_weights(7, dims)

    def build():
        layers = [rt.Identity()]
        for l, (w, b) in enumerate(W):
            layers.append(rt.Linear.new_with_kernel(dims[l], dims[l + 1], Fixed(w, b)))
            if l + 1 < len(W):
                layers.append(rt.ReLU())
        return rt.sequential(*layers).to(ctx)

    X, T = synth.mnist_like(7, 0, 8 * 3, features=20, classes=5, zero_fraction=0.5)
    xd, td = ctx.empty(8, 20), ctx.empty(8, 5)
    loss_fn, opt = rt.CrossEntropyLoss(), rt.SGD.new(0.05)

    def step(model, slot):
        pred = model.forward(xd)
        loss_fn.forward_async(pred, td, slot)
        model.backward(loss_fn.backward(), need_input_grad=False)
        opt.step(model)

    eager, graphed = build(), build()
    eager_losses = []
    for s in range(3):
        xd.upload(X[s * 8:(s + 1) * 8]); td.upload(T[s * 8:(s + 1) * 8])
        step(eager, 1)
        eager_losses.append(loss_fn.result(1)[0])
    # Nothing is allocated from the driver while recording, so the same step runs once,
    # unrecorded, directly before the capture; that run moves the weights, which are put
    # back before the replays (recording itself executes nothing).
    xd.upload(X[:8]); td.upload(T[:8])
    step(graphed, 2)
    with ctx.capture() as cap:
        step(graphed, 2)
    for lin, (w, b) in zip([l for l in graphed.layers if isinstance(l, rt.Linear)], W):
        lin.weight.upload(w); lin.bias.upload(b)
    losses = []
    for s in range(3):
        xd.upload(X[s * 8:(s + 1) * 8]); td.upload(T[s * 8:(s + 1) * 8])
        cap.graph.launch()
        losses.append(loss_fn.result(2)[0])
    assert losses == eager_losses
    for a, b in zip(eager.parameters(), graphed.parameters()):
        assert np.array_equal(a.parm.numpy(), b.parm.numpy())
    cap.graph.destroy()


def test_graph_keeps_its_blocks_out_of_the_allocator():
    """Nothing is allocated from the driver while recording; the blocks the recorded kernels
    address stay out of the cache until the graph is destroyed, so a later tensor can never be
    handed memory that a replay overwrites."""
    c = rt.Context(0)
    try:
        x = c.tensor(np.full((64, 64), 2.0))

        def work():
            a = c.empty(64, 64)                       # an intermediate: written, read, dropped
            c._check(c._lib.rst_relu_forward(c.handle, x.handle, a.handle))
            out = c.empty(64, 64)
            c._check(c._lib.rst_relu_forward(c.handle, a.handle, out.handle))
            return a.data_ptr(), out

        # recording without a warm cache: no driver allocation is made, the call fails cleanly
        c.empty_cache()
        with pytest.raises(rt.RstError) as e:
            with c.capture():
                work()
        assert e.value.status == _lib.RST_ERR_STATE and "directly before" in str(e.value)
        # the unrecorded run fills the cache, the recorded one is served from it
        _, out = work()
        del out
        allocs = c.memory_stats()["driver_allocs"]
        with c.capture() as cap:
            a_ptr, out = work()
        assert c.memory_stats()["driver_allocs"] == allocs
        out_ptr = out.data_ptr()
        # while the graph lives neither block is handed out again, even after `out` is dropped
        del out
        later = [c.empty(64, 64) for _ in range(6)]
        assert a_ptr not in {t.data_ptr() for t in later} and out_ptr not in {t.data_ptr() for t in later}
        for t in later:
            t.fill(-1.0)
        cap.graph.launch()
        c.synchronize()
        for t in later:
            assert np.array_equal(t.numpy(), np.full((64, 64), -1.0))     # the replay wrote elsewhere
        in_use = c.memory_stats()["in_use"]
        cap.graph.destroy()
        assert c.memory_stats()["in_use"] == in_use - 2 * 64 * 64 * 8      # both blocks are back in the cache
        again = {c.empty(64, 64).data_ptr() for _ in range(1)}
        assert again & {a_ptr, out_ptr}
    finally:
        c.close()


@pytest.mark.parametrize("B,cin,cout,fused_copy", [
    (2048, 1280, 640, True),     # 160 large tiles, no split: dX and its transposed copy from one kernel
    (3000, 4000, 4100, True),    # 768 large tiles: the transposed copy of the tail's tiles comes from the fix-up
    (2048, 2048, 2048, False),   # 256 large tiles split K four ways: separate transpose kernel
    (96, 64, 40, False),         # small tiles
    (50, 33, 21, False),         # odd widths: plain-load kernel
])
def test_linear_backward_with_transposed_companions(ctx, oc, B, cin, cout, fused_copy):
    rng = np.random.default_rng(B + cin)
    X = np.maximum(rng.standard_normal((B, cin)), 0.0)
    W, dY = rng.standard_normal((cout, cin)) / np.sqrt(cin), rng.standard_normal((B, cout))
    xd, wd, gd = ctx.tensor(X), ctx.tensor(W), ctx.tensor(dY)
    gt = ctx.empty(cout, B)
    ctx._check(ctx._lib.rst_transpose(ctx.handle, gd.handle, gt.handle))
    assert np.array_equal(gt.numpy(), dY.T)
    dW, db, dX, dXt = ctx.empty(cout, cin), ctx.empty(1, cout), ctx.empty(B, cin), ctx.empty(cin, B)
    before = ctx.launch_count()
    ctx._check(ctx._lib.rst_linear_backward_t(ctx.handle, gd.handle, gt.handle, xd.handle, wd.handle, xd.handle,
                                              dW.handle, db.handle, dX.handle, dXt.handle))
    launches = ctx.launch_count() - before
    want_dW, want_db, want_dX = oc.linear_backward(dY, X, W)
    want_dX = want_dX * (X > 0.0)
    assert rel_err(dW.numpy(), want_dW) < REL_TOL and rel_err(db.numpy(), want_db) < REL_TOL
    assert rel_err(dX.numpy(), want_dX) < REL_TOL
    assert np.array_equal(dXt.numpy(), dX.numpy().T)                     # the same values, transposed
    # against the plain entry point: another kernel variant, same sums in another order
    dW2, db2, dX2 = ctx.empty(cout, cin), ctx.empty(1, cout), ctx.empty(B, cin)
    before = ctx.launch_count()
    ctx._check(ctx._lib.rst_linear_backward(ctx.handle, gd.handle, xd.handle, wd.handle, xd.handle,
                                            dW2.handle, db2.handle, dX2.handle))
    plain_launches = ctx.launch_count() - before
    assert rel_err(dX.numpy(), dX2.numpy()) < 1e-13 and np.array_equal(dW.numpy(), dW2.numpy())
    if fused_copy:
        assert launches == plain_launches                                # no transpose launch
    # without the companions the call is rst_linear_backward; dX_t alone is honoured too
    dX3, dXt3 = ctx.empty(B, cin), ctx.empty(cin, B)
    ctx._check(ctx._lib.rst_linear_backward_t(ctx.handle, gd.handle, None, xd.handle, wd.handle, xd.handle,
                                              dW.handle, db.handle, dX3.handle, dXt3.handle))
    assert np.array_equal(dX3.numpy(), dX2.numpy()) and np.array_equal(dXt3.numpy(), dX2.numpy().T)
    # shape errors: a companion that is not (cols, rows) of its tensor
    wrong = ctx.empty(cout + 1, B)
    assert ctx._lib.rst_linear_backward_t(ctx.handle, gd.handle, wrong.handle, xd.handle, wd.handle, None,
                                          dW.handle, db.handle, dX.handle, None) == _lib.RST_ERR_SHAPE
    assert ctx._lib.rst_linear_backward_t(ctx.handle, gd.handle, gt.handle, xd.handle, wd.handle, None,
                                          dW.handle, db.handle, dX.handle, wrong.handle) == _lib.RST_ERR_SHAPE
    assert ctx._lib.rst_transpose(ctx.handle, gd.handle, wrong.handle) == _lib.RST_ERR_SHAPE
