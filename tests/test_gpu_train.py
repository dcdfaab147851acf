"""Whole training steps through the public API against the CPU restatement: the
committed golden steps, the README model on the MNIST-shaped stream, and
size-independent properties at benchmark sizes."""
import numpy as np
import pytest

import rstorch_b200 as rt
from conftest import REL_TOL, rel_err
from rstorch_b200 import synth

pytestmark = pytest.mark.gpu


class Fixed(rt.InitParameters):
    def __init__(self, w, b):
        self.w, self.b = w, b

    def weight(self, i, o):
        return self.w

    def bias(self, i, o):
        return self.b


def build_mlp(ctx, dims, weights, identity=True):
    layers = [rt.Identity()] if identity else []
    for l, (w, b) in enumerate(weights):
        layers.append(rt.Linear.new_with_kernel(dims[l], dims[l + 1], Fixed(w, b)))
        if l + 1 < len(weights):
            layers.append(rt.ReLU())
    return rt.sequential(*layers).to(ctx)


def linears(model):
    return [l for l in model.layers if isinstance(l, rt.Linear)]


def test_golden_steps(ctx, golden_steps):
    g = golden_steps
    dims = g["dims"].tolist()
    L, B, steps, lr = len(dims) - 1, int(g["batch"]), int(g["steps"]), float(g["lr"])
    model = build_mlp(ctx, dims, [(g[f"W0_{l}"], g[f"b0_{l}"]) for l in range(L)])
    loss_fn, opt = rt.CrossEntropyLoss(), rt.SGD.new(lr)
    for s in range(steps):
        x, t = ctx.tensor(g["X"][s * B:(s + 1) * B]), ctx.tensor(g["T"][s * B:(s + 1) * B])
        pred = model.forward(x)
        loss = loss_fn.forward(pred, t)
        acc = rt.accuracy(pred, t)
        assert rel_err(pred.numpy(), g[f"logits_{s}"]) < REL_TOL
        assert abs(loss - float(g[f"loss_{s}"])) <= REL_TOL * abs(float(g[f"loss_{s}"]))
        assert acc == float(g[f"acc_{s}"]) == loss_fn.last_accuracy
        model.backward(loss_fn.backward())
        for l, lin in enumerate(linears(model)):
            assert rel_err(lin.grad_weight.numpy(), g[f"dW_{s}_{l}"]) < REL_TOL
            assert rel_err(lin.grad_bias.numpy(), g[f"db_{s}_{l}"]) < REL_TOL
        opt.step(model)
        for l, lin in enumerate(linears(model)):
            assert rel_err(lin.weight.numpy(), g[f"W_{s}_{l}"]) < REL_TOL
            assert rel_err(lin.bias.numpy(), g[f"b_{s}_{l}"]) < REL_TOL


@pytest.mark.parametrize("batch,steps,chunk", [(32, 1875, 1875), (4096, 200, 25)])
def test_readme_model_full_length_trajectory(ctx, oc, batch, steps, chunk):
    """784-100-100-10, lr 0.01, at the step counts of the two benchmark configurations: one
    epoch of 60000 samples at batch 32 (1875 steps) and 200 steps at batch 4096 (819,200
    samples drawn fresh from the stream, never cycled).  Both sides run freely from the same
    initial weights; every step compares the loss, the accuracy (bit-exact), every gradient
    and every updated weight.  The smallest gap between the two largest logits of any row is
    tracked: the arg-max can only be guaranteed while it exceeds the logits' error."""
    dims = [784, 100, 100, 10]
    w_cpu = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(0, dims)]
    model = build_mlp(ctx, dims, w_cpu)
    loss_fn, opt = rt.CrossEntropyLoss(), rt.SGD.new(0.01)
    min_gap, worst, s = np.inf, 0.0, -1
    for first in range(0, steps, chunk):
        n = min(chunk, steps - first)
        X, T = synth.mnist_like(0, first * batch, n * batch)
        ds = rt.ArrayDataset(X, T)
        dl = rt.DataLoader(ds, batch, False, rt.SequentialSampler(len(ds)), ctx, slots=3)
        for k, (x, t) in enumerate(dl.iter_array()):
            s = first + k
            pred = model.forward(x)
            loss = loss_fn.forward(pred, t)
            acc = rt.accuracy(pred, t)
            logits = pred.numpy()
            model.backward(loss_fn.backward(), need_input_grad=False)
            opt.step(model)
            xb, tb = X[k * batch:(k + 1) * batch], T[k * batch:(k + 1) * batch]
            losses, accs, grads = oc.mlp_train(dims, w_cpu, xb, tb, batch, 1, 0.01, skip_first_dx=True)
            top2 = np.partition(logits, -2, axis=1)[:, -2:]
            min_gap = min(min_gap, float((top2[:, 1] - top2[:, 0]).min()))
            assert abs(loss - losses[0]) <= REL_TOL * abs(losses[0]), s
            assert acc == accs[0] == loss_fn.last_accuracy, (s, min_gap)
            for l, lin in enumerate(linears(model)):
                errs = (rel_err(lin.grad_weight.numpy(), grads[l][0]), rel_err(lin.grad_bias.numpy(), grads[l][1]),
                        rel_err(lin.weight.numpy(), w_cpu[l][0]), rel_err(lin.bias.numpy(), w_cpu[l][1]))
                worst = max(worst, *errs)
                assert max(errs) < REL_TOL, (s, l, errs)
        dl.close()
    assert s == steps - 1
    assert min_gap > 1e-9, min_gap          # no row's arg-max hung on less than the error bar
    print(f"batch {batch}: {steps} steps, worst relative error {worst:.3e}, smallest top-2 logit gap {min_gap:.3e}")
    ctx.check_device()


def test_basic_model_step_and_predict(ctx, oc):
    """`BasicModel::step` / `predict` (model.rs:19-31) over the device path."""
    dims = [20, 16, 5]
    w_cpu = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(4, dims)]
    model = rt.BasicModel.new(build_mlp(ctx, dims, w_cpu), rt.CrossEntropyLoss(), rt.SGD.new(0.05))
    X, T = synth.mnist_like(4, 0, 24, features=20, classes=5, zero_fraction=0.3)
    x, t = ctx.tensor(X), ctx.tensor(T)
    before = model.predict(x).numpy()
    assert rel_err(before, oc.linear_forward(oc.relu_forward(oc.linear_forward(X, *w_cpu[0])), *w_cpu[1])) < REL_TOL
    model.step(x, t)
    oc.mlp_train(dims, w_cpu, X, T, 24, 1, 0.05)
    for lin, (w, b) in zip(linears(model.module), w_cpu):
        assert rel_err(lin.weight.numpy(), w) < REL_TOL and rel_err(lin.bias.numpy(), b) < REL_TOL
    after = model.predict(x).numpy()
    assert not np.array_equal(before, after)


def test_fused_and_unfused_paths_agree(ctx):
    """Calling the layers one by one (no peephole fusion) gives the same step as Sequential."""
    dims = [64, 48, 40, 10]
    W = synth.mlp_weights(3, dims)
    X, T = synth.gaussian_batch(3, 0, 0, 96, 64, 10, 96)
    fused, plain = build_mlp(ctx, dims, W), build_mlp(ctx, dims, W)
    lf1, lf2 = rt.CrossEntropyLoss(), rt.CrossEntropyLoss()
    x, t = ctx.tensor(X), ctx.tensor(T)
    l1 = lf1.forward(fused.forward(x), t)
    dx1 = fused.backward(lf1.backward())
    h = x
    for layer in plain.layers:
        h = layer.forward(h)
    l2 = lf2.forward(h, t)
    g = lf2.backward()
    for layer in reversed(plain.layers):
        g = layer.backward(g)
    assert l1 == l2
    assert np.array_equal(dx1.numpy(), g.numpy())
    # the container sends all dW products out in one grouped launch, which may cut the batch
    # dimension into other split-K pieces than a single product does: same sums, other order
    for a, b in zip(fused.parameters(), plain.parameters()):
        assert rel_err(a.grad.numpy(), b.grad.numpy()) < 1e-13


def test_wide_layer_sampled_entries_at_benchmark_size(ctx):
    """8192 x 4096 x 4096 (the wide-MLP layer): a CPU restatement of the full product is
    too slow, so random output entries are recomputed as long-double dot products, and the
    linearity of the layer in its input is checked on the whole output."""
    rng = np.random.default_rng(0)
    B, cin, cout = 8192, 4096, 4096
    X = synth.normal(synth.stream_key(0, "t.x"), B * cin).reshape(B, cin)
    W = synth.normal(synth.stream_key(0, "t.w"), cout * cin, std=1 / 64).reshape(cout, cin)
    b = np.zeros((1, cout))
    lin = rt.Linear.new_with_kernel(cin, cout, Fixed(W, b))
    xd = ctx.tensor(X)
    y = lin.forward(xd).numpy()
    dY = synth.normal(synth.stream_key(0, "t.g"), B * cout).reshape(B, cout)
    dx = lin.backward(ctx.tensor(dY)).numpy()
    dW = lin.grad_weight.numpy()
    db = lin.grad_bias.numpy()
    ld = np.longdouble
    scale_y, scale_dx, scale_dw = np.abs(y).max(), np.abs(dx).max(), np.abs(dW).max()
    for _ in range(64):
        r, c, k = rng.integers(0, B), rng.integers(0, cout), rng.integers(0, cin)
        assert abs(y[r, c] - float(np.dot(X[r].astype(ld), W[c].astype(ld)))) < REL_TOL * scale_y
        assert abs(dx[r, k] - float(np.dot(dY[r].astype(ld), W[:, k].astype(ld)))) < REL_TOL * scale_dx
        assert abs(dW[c, k] - float(np.dot(dY[:, c].astype(ld), X[:, k].astype(ld)) / B)) < REL_TOL * scale_dw
    assert rel_err(db, dY.sum(axis=0, keepdims=True) / B) < REL_TOL
    # linearity: forward(2x) == 2*forward(x) exactly (powers of two do not round), bias is zero
    y2 = lin.forward(ctx.tensor(2.0 * X)).numpy()
    assert np.array_equal(y2, 2.0 * y)
    ctx.check_device()


def test_wide_mlp_full_size_steps(ctx, oc):
    """The wide-MLP workload at its own size (1024-4096-4096-4096-1000, batch 8192, a fresh
    batch per step): three free-running steps against the CPU restatement, every gradient
    and updated weight at every step."""
    dims, batch, steps = [1024, 4096, 4096, 4096, 1000], 8192, 3
    w_cpu = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(0, dims)]
    model = build_mlp(ctx, dims, w_cpu, identity=False)
    loss_fn, opt = rt.CrossEntropyLoss(), rt.SGD.new(0.01)
    for s in range(steps):
        X, T = synth.gaussian_batch(0, s, 0, batch, dims[0], dims[-1], batch)
        pred = model.forward(ctx.tensor(X))
        loss = loss_fn.forward(pred, ctx.tensor(T))
        model.backward(loss_fn.backward(), need_input_grad=False)
        opt.step(model)
        losses, accs, grads = oc.mlp_train(dims, w_cpu, X, T, batch, 1, 0.01, skip_first_dx=True)
        assert abs(loss - losses[0]) <= REL_TOL * abs(losses[0]), s
        assert loss_fn.last_accuracy == accs[0], s
        for l, lin in enumerate(linears(model)):
            assert rel_err(lin.grad_weight.numpy(), grads[l][0]) < REL_TOL, (s, l)
            assert rel_err(lin.grad_bias.numpy(), grads[l][1]) < REL_TOL, (s, l)
            assert rel_err(lin.weight.numpy(), w_cpu[l][0]) < REL_TOL, (s, l)
            assert rel_err(lin.bias.numpy(), w_cpu[l][1]) < REL_TOL, (s, l)
    ctx.check_device()


def test_deep_mlp_reduced_width_trajectory(ctx, oc):
    """The deep-MLP topology (input, ten Linear layers with ReLU between them, 1000 classes)
    at reduced width and batch: three free-running steps against the restatement."""
    dims, batch, steps = [256] + [512] * 9 + [1000], 512, 3
    w_cpu = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(2, dims)]
    model = build_mlp(ctx, dims, w_cpu, identity=False)
    loss_fn, opt = rt.CrossEntropyLoss(), rt.SGD.new(0.01)
    for s in range(steps):
        X, T = synth.gaussian_batch(2, s, 0, batch, dims[0], dims[-1], batch)
        loss = loss_fn.forward(model.forward(ctx.tensor(X)), ctx.tensor(T))
        model.backward(loss_fn.backward(), need_input_grad=False)
        opt.step(model)
        losses, accs, grads = oc.mlp_train(dims, w_cpu, X, T, batch, 1, 0.01, skip_first_dx=True)
        assert abs(loss - losses[0]) <= REL_TOL * abs(losses[0]) and loss_fn.last_accuracy == accs[0]
        for l, lin in enumerate(linears(model)):
            assert rel_err(lin.grad_weight.numpy(), grads[l][0]) < REL_TOL, (s, l)
            assert rel_err(lin.weight.numpy(), w_cpu[l][0]) < REL_TOL, (s, l)
