"""TEST INFRASTRUCTURE: numpy twin of the CPU restatement (small cases only).

Each function restates one reference function with numpy array expressions that
mirror the ndarray expressions of the Rust source line by line; it cross-checks
the C++ restatement and generates the committed golden fixtures.
"""
from __future__ import annotations

import numpy as np

F64_MIN = -np.finfo(np.float64).max


def linear_forward(X, W, b=None):
    """src/module/linear.rs:43-57: input.dot(&weight.t()) then x += bias."""
    y = X @ W.T
    if b is not None:
        y = y + b.reshape(1, -1)
    return y


def linear_backward(dY, X, W):
    """src/module/linear.rs:60-69: (gradient.t().dot(prev_input)/n, sum_axis(0)/n as (1,out), gradient.dot(weight))."""
    n = float(X.shape[0])
    dW = (dY.T @ X) / n
    db = (dY.sum(axis=0) / n)[None, :]
    dX = dY @ W
    return dW, db, dX


def relu_forward(x):
    """src/module/activation/relu.rs:21: x.max(0.0) with f64::max (NaN -> 0)."""
    return np.where(np.isnan(x), 0.0, np.maximum(x, 0.0))


def relu_backward(dy, xpre):
    """src/module/activation/relu.rs:26: gradient * f64::from(x > 0.0)."""
    return dy * (xpre > 0.0).astype(np.float64)


def softmax(x):
    """src/module/activation/softmax.rs:45-53 (axis 1)."""
    m = np.maximum(np.max(np.where(np.isnan(x), F64_MIN, x), axis=1, keepdims=True), F64_MIN)
    e = np.exp(x - m)
    return e / e.sum(axis=1, keepdims=True)


def softmax_axis(x, axis):
    """src/module/activation/softmax.rs:45-53 for either axis."""
    m = np.maximum(np.max(np.where(np.isnan(x), F64_MIN, x), axis=axis, keepdims=True), F64_MIN)
    e = np.exp(x - m)
    return e / e.sum(axis=axis, keepdims=True)


def softmax_module_backward(output, gradient):
    """Softmax::backward, src/module/activation/softmax.rs:62-75: jacobian = -(outputᵀ·output);
    each diagonal element el becomes -el and then el·(1 - el); result = gradient · jacobian."""
    jac = -(output.T @ output)
    d = -np.diag(jac)
    jac[np.diag_indices_from(jac)] = d * (1.0 - d)
    return gradient @ jac


def xent_forward(pred, truth):
    """src/loss/cross_entropy.rs:34-42 -> (loss, cached softmax)."""
    p = softmax(pred)
    with np.errstate(divide="ignore", invalid="ignore"):
        loss = -(truth * np.log(p)).sum() / float(pred.shape[0])
    return float(loss), p


def xent_backward(p, truth):
    """src/loss/cross_entropy.rs:45-47."""
    return -(truth - p)


def sgd_step(p, g, lr):
    """src/optim/sgd.rs:23: parm - (lr * grad); numpy rounds the product, then the difference."""
    return p - (lr * g)


def argmax(x):
    """src/utils.rs:44-53: first maximum wins, replace only on strict `>`."""
    out = np.zeros(x.shape[0], dtype=np.int64)
    for r in range(x.shape[0]):
        best, bv = 0, x[r, 0]
        for c in range(1, x.shape[1]):
            if x[r, c] > bv:
                best, bv = c, x[r, c]
        out[r] = best
    return out


def accuracy(pred, truth):
    """src/utils.rs:55-65."""
    return float((argmax(pred) == argmax(truth)).sum()) / float(pred.shape[0])


def normalize_zero_one(x):
    """src/utils.rs:5-18 for a u8 sample: max and min by `Ord` on the source type, then
    `(R::from(v) - min) / (max - min)` in f64 (0/0 = NaN when the sample is constant)."""
    mx, mn = float(x.max()), float(x.min())
    with np.errstate(divide="ignore", invalid="ignore"):
        return (x.astype(np.float64) - mn) / (mx - mn)


def flatten(x):
    """src/utils.rs:30-35: elements in logical (row-major) order."""
    return np.ascontiguousarray(x).reshape(-1)


def one_hot(label, n):
    """src/utils.rs:38-42."""
    out = np.zeros(n, dtype=np.float64)
    out[int(label)] = 1.0
    return out


def iter_array_batch(images, labels, indices, classes):
    """One batch of `ArrayDataLoaderIter::next` (src/data/data_loader.rs:192-207) over the
    README transform `(flatten(normalize_zero_one(x)), one_hot(y, classes))` (README.md:44)."""
    X = np.stack([flatten(normalize_zero_one(images[i])) for i in indices])
    T = np.stack([one_hot(labels[i], classes) for i in indices])
    return X, T


def epoch_permutation(seed: int, n: int) -> np.ndarray:
    """Host mirror of the seeded epoch order that stands in for `Shuffler::shuffle`
    (src/data/dataset/shuffler.rs:15-25, unseedable in the reference): position i maps to
    sample perm(i), a four-round Feistel network over the smallest even bit width that covers
    n, cycle-walked below n; round function splitmix64(seed + round·φ64 + right half)."""
    M64 = (1 << 64) - 1
    bits = 2
    while bits < 62 and (1 << bits) < n:
        bits += 2
    half = bits // 2
    mask = (1 << half) - 1

    def mix(z: int) -> int:
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        return z ^ (z >> 31)

    out = np.empty(n, dtype=np.int64)
    for i in range(n):
        v = i
        while True:
            l, r = v >> half, v & mask
            for rnd in range(4):
                f = mix((seed + 0x9E3779B97F4A7C15 * (rnd + 1) + r) & M64) & mask
                l, r = r, l ^ f
            v = (l << half) | r
            if v < n:
                break
        out[i] = v
    return out


def mlp_step(weights, X, T, lr, skip_first_dx=False):
    """One step in the order of src/model.rs:19-27 for Linear,ReLU,...,Linear.
    Returns (loss, acc, grads, new_weights, logits)."""
    acts, pres = [X], []
    for l, (W, b) in enumerate(weights):
        z = linear_forward(acts[-1], W, b)
        pres.append(z)
        acts.append(relu_forward(z) if l + 1 < len(weights) else z)
    logits = pres[-1]
    loss, p = xent_forward(logits, T)
    acc = accuracy(logits, T)
    g = xent_backward(p, T)
    grads = [None] * len(weights)
    for l in range(len(weights) - 1, -1, -1):
        W, _ = weights[l]
        dW, db, dX = linear_backward(g, acts[l], W)
        grads[l] = (dW, db)
        if l > 0:
            g = relu_backward(dX, pres[l - 1])
    new = [(sgd_step(W, dW, lr), sgd_step(b, db, lr)) for (W, b), (dW, db) in zip(weights, grads)]
    return loss, acc, grads, new, logits
