"""The CPU restatement against the reference's own known-answer tests, against its
numpy twin, and against the committed golden steps.  No GPU needed."""
import numpy as np
import pytest

from conftest import REL_TOL, rel_err
from oracle import oracle_np as on


def A(x):
    return np.array(x, dtype=np.float64)


# ---- vectors from the reference's unit tests ------------------------------------
def test_kat_linear_forward(kat, oc):
    k = kat["linear_forward"]
    y = oc.linear_forward(A(k["input"]), A(k["weight"]), A(k["bias"]))
    assert y.shape == (3, 1)
    assert np.max(np.abs(y - A(k["expected"]))) <= kat["tolerance"]
    assert np.array_equal(y, on.linear_forward(A(k["input"]), A(k["weight"]), A(k["bias"])))


def test_kat_linear_backward(kat, oc):
    k = kat["linear_backward"]
    dW, db, dX = oc.linear_backward(A(k["gradient"]), A(k["input"]), A(k["weight"]))
    assert dW.shape == A(k["weight"]).shape and db.shape == A(k["bias"]).shape   # linear.rs:113-121
    tol = kat["tolerance"]
    assert np.max(np.abs(dW - A(k["expected_grad_weight"]))) <= tol
    assert np.max(np.abs(db - A(k["expected_grad_bias"]))) <= tol
    assert np.max(np.abs(dX - A(k["expected_grad_input"]))) <= tol


def test_kat_relu(kat, oc):
    f, b = kat["relu_forward"], kat["relu_backward"]
    assert np.array_equal(oc.relu_forward(A(f["input"])), A(f["expected"]))
    assert np.array_equal(oc.relu_backward(A(b["gradient"]), A(b["input"])), A(b["expected"]))


def test_kat_softmax_rows(kat, oc):
    k = kat["softmax_rows_sum_to_one"]
    p, nan_rows = oc.softmax(A(k["input"]))
    assert nan_rows == 0
    assert np.max(np.abs(p.sum(axis=1) - A(k["expected_row_sums"]))) <= kat["tolerance"]
    assert abs(p.sum() - k["expected_total"]) <= 4 * np.finfo(float).eps


def test_kat_softmax_module(kat):
    k = kat["softmax_axis0_columns_sum_to_one"]
    p = on.softmax_axis(A(k["input"]), 0)
    assert np.max(np.abs(p.sum(axis=0) - A(k["expected_column_sums"]))) <= kat["tolerance"]
    assert abs(p.sum() - k["expected_total"]) <= 4 * np.finfo(float).eps
    b = kat["softmax_module_backward"]
    out = on.softmax_axis(A(b["input"]), 1)
    got = on.softmax_module_backward(out, A(b["gradient"]))
    assert np.max(np.abs(got - A(b["expected"]))) <= b["tolerance"]
    assert np.array_equal(on.softmax_axis(A(b["input"]), 1), on.softmax(A(b["input"])))


def test_kat_sgd_zero_gradient(kat, oc):
    k = kat["sgd_zero_gradient"]
    w = np.array([[0.3, -0.2], [1.5, 2.5]])
    assert np.array_equal(oc.sgd_step(w, A(k["gradient"]), k["lr"]), w)


# ---- C++ restatement against the numpy twin ---------------------------------------
@pytest.mark.parametrize("B,cin,cout", [(1, 1, 1), (3, 2, 1), (32, 784, 100), (17, 33, 9), (64, 100, 10)])
def test_linear_matches_numpy(oc, B, cin, cout):
    rng = np.random.default_rng(B * 1000 + cin)
    X, W, b = rng.standard_normal((B, cin)), rng.standard_normal((cout, cin)), rng.standard_normal((1, cout))
    dY = rng.standard_normal((B, cout))
    assert rel_err(oc.linear_forward(X, W, b), on.linear_forward(X, W, b)) < 1e-13
    for got, want in zip(oc.linear_backward(dY, X, W), on.linear_backward(dY, X, W)):
        assert rel_err(got, want) < 1e-13


def test_precise_gemm_bounds_plain_gemm(oc):
    rng = np.random.default_rng(5)
    X, W = rng.standard_normal((40, 3000)), rng.standard_normal((24, 3000))
    plain, precise = oc.linear_forward(X, W), oc.linear_forward(X, W, precise=True)
    assert rel_err(plain, precise) < 1e-13


def test_softmax_xent_matches_numpy(oc):
    rng = np.random.default_rng(3)
    for C in (2, 10, 37, 1000):
        x = rng.standard_normal((19, C)) * 5
        t = np.eye(C)[rng.integers(0, C, 19)]
        loss_c, p_c, nan_rows = oc.xent_forward(x, t)
        loss_n, p_n = on.xent_forward(x, t)
        assert nan_rows == 0
        assert rel_err(p_c, p_n) < 1e-14 and abs(loss_c - loss_n) <= 1e-13 * abs(loss_n)
        assert np.array_equal(oc.xent_backward(p_c, t), on.xent_backward(p_c, t))


def test_xent_underflow_gives_nan_like_the_reference(oc):
    # cross_entropy.rs:38 multiplies truth by ln(p) for every class: p underflows to 0 for a
    # logit gap beyond ~745, ln(0) = -inf and 0 * -inf = NaN.
    x = np.array([[0.0, -800.0]])
    t = np.array([[1.0, 0.0]])
    loss, p, _ = oc.xent_forward(x, t)
    assert p[0, 1] == 0.0 and np.isnan(loss)
    assert np.isnan(on.xent_forward(x, t)[0])


def test_softmax_counts_nan_rows(oc):
    x = np.array([[1.0, np.nan], [0.0, 1.0], [np.nan, np.nan]])
    assert oc.softmax(x)[1] == 2


def test_sgd_rounds_product_then_difference(oc):
    rng = np.random.default_rng(11)
    p, g = rng.standard_normal(4097), rng.standard_normal(4097) * 1e-3
    want = p - (0.01 * g)                      # numpy: two roundings, like ndarray
    assert np.array_equal(oc.sgd_step(p, g, 0.01), want)
    fused = np.array([float(np.float64(np.longdouble(a) - np.longdouble(0.01) * np.longdouble(b)))
                      for a, b in zip(p, g)])
    assert not np.array_equal(fused, want)     # a single-rounding update differs somewhere


def test_argmax_first_maximum_wins(oc):
    x = np.array([[1.0, 3.0, 3.0, 2.0], [5.0, 5.0, 5.0, 5.0], [np.nan, 9.0, 1.0, 0.0],
                  [1.0, np.nan, 7.0, 7.0], [-np.inf, -np.inf, np.nan, -np.inf]])
    assert oc.argmax(x).tolist() == [1, 0, 0, 2, 0]
    assert on.argmax(x).tolist() == [1, 0, 0, 2, 0]
    t = np.eye(4)[[1, 0, 3, 2, 0]]
    assert oc.accuracy(x, t) == pytest.approx(4 / 5)


def test_readme_transform_restatement():
    x = np.array([[10, 60], [110, 210]], dtype=np.uint8)
    assert on.flatten(on.normalize_zero_one(x)).tolist() == [0.0, 0.25, 0.5, 1.0]
    assert np.isnan(on.normalize_zero_one(np.full((2, 2), 7, dtype=np.uint8))).all()     # 0 / 0
    assert on.one_hot(2, 4).tolist() == [0.0, 0.0, 1.0, 0.0]
    with pytest.raises(IndexError):
        on.one_hot(4, 4)
    from rstorch_b200 import synth
    images, labels = synth.mnist_like_u8(0, 0, 64)
    assert images.shape == (64, 28, 28) and images.dtype == np.uint8 and labels.max() < 10
    assert 0.78 < (images == 0).mean() < 0.84
    X, T = on.iter_array_batch(images, labels, [5, 3], 10)
    assert X.shape == (2, 784) and T.shape == (2, 10) and X.max() == 1.0 and X.min() == 0.0
    assert T[0].argmax() == labels[5] and T.sum() == 2.0


# ---- committed golden steps ------------------------------------------------------------
def test_golden_steps_cpp(oc, golden_steps):
    g = golden_steps
    dims = g["dims"].tolist()
    L, B, steps, lr = len(dims) - 1, int(g["batch"]), int(g["steps"]), float(g["lr"])
    weights = [(g[f"W0_{l}"].copy(), g[f"b0_{l}"].copy()) for l in range(L)]
    for s in range(steps):
        xb, tb = g["X"][s * B:(s + 1) * B], g["T"][s * B:(s + 1) * B]
        losses, accs, grads = oc.mlp_train(dims, weights, xb, tb, B, 1, lr)
        assert abs(losses[0] - float(g[f"loss_{s}"])) <= REL_TOL * abs(float(g[f"loss_{s}"]))
        assert accs[0] == float(g[f"acc_{s}"])
        for l in range(L):
            assert rel_err(grads[l][0], g[f"dW_{s}_{l}"]) < REL_TOL
            assert rel_err(grads[l][1], g[f"db_{s}_{l}"]) < REL_TOL
            assert rel_err(weights[l][0], g[f"W_{s}_{l}"]) < REL_TOL
            assert rel_err(weights[l][1], g[f"b_{s}_{l}"]) < REL_TOL


def test_golden_steps_numpy(golden_steps):
    g = golden_steps
    dims = g["dims"].tolist()
    L, B, steps, lr = len(dims) - 1, int(g["batch"]), int(g["steps"]), float(g["lr"])
    weights = [(g[f"W0_{l}"], g[f"b0_{l}"]) for l in range(L)]
    for s in range(steps):
        loss, acc, grads, weights, logits = on.mlp_step(weights, g["X"][s * B:(s + 1) * B],
                                                        g["T"][s * B:(s + 1) * B], lr)
        assert abs(loss - float(g[f"loss_{s}"])) <= 1e-12 * abs(loss)
        assert rel_err(logits, g[f"logits_{s}"]) < 1e-12


def test_multistep_and_skip_first_dx_do_not_change_results(oc):
    from rstorch_b200 import synth
    dims = [784, 100, 100, 10]
    X, T = synth.mnist_like(0, 0, 96)
    w1 = [(w.copy(), b.copy()) for w, b in synth.mlp_weights(0, dims)]
    w2 = [(w.copy(), b.copy()) for w, b in w1]
    l1, a1, g1 = oc.mlp_train(dims, w1, X, T, 32, 3, 0.01, skip_first_dx=False)
    l2, a2, g2 = oc.mlp_train(dims, w2, X, T, 32, 3, 0.01, skip_first_dx=True)
    assert np.array_equal(l1, l2) and np.array_equal(a1, a2)
    for (wa, ba), (wb, bb) in zip(w1, w2):
        assert np.array_equal(wa, wb) and np.array_equal(ba, bb)
    assert 2.0 < l1[0] < 2.8          # ~ln(10) at initialisation


def test_oracle_generator_matches_the_library_generator_bit_for_bit():
    """The benchmark's CPU arm draws its inputs from the oracle's own generator; both
    generators restate the same streams (splitmix64 words, 53-bit uniforms, Box-Muller)."""
    from oracle import oracle_synth as osy
    from rstorch_b200 import synth
    for seed, purpose, index in [(0, "weight", 0), (3, "gaussian.x", 0), (7, "x", 5)]:
        k = synth.stream_key(seed, purpose, index)
        assert k == osy.stream_key(seed, purpose, index)
        assert np.array_equal(synth.uniform(k, 5000, offset=123), osy.uniform(k, 5000, offset=123))
        assert np.array_equal(synth.normal(k, 5000, std=0.02, mean=0.5, offset=99),
                              osy.normal(k, 5000, std=0.02, mean=0.5, offset=99))
    for a, b in zip(synth.mnist_like(0, 10, 64), osy.mnist_like(0, 10, 64)):
        assert np.array_equal(a, b)
    for a, b in zip(synth.gaussian_batch(0, 2, 16, 48, 24, 9, 128), osy.gaussian_batch(0, 2, 16, 48, 24, 9, 128)):
        assert np.array_equal(a, b)
    for (wa, ba), (wb, bb) in zip(synth.mlp_weights(0, [64, 48, 10]), osy.mlp_weights(0, [64, 48, 10])):
        assert np.array_equal(wa, wb) and np.array_equal(ba, bb)


def test_epoch_permutation_mirror_is_a_seeded_bijection():
    for n in (1, 2, 3, 17, 256, 1000, 60000):
        p = on.epoch_permutation(11, n)
        assert np.array_equal(np.sort(p), np.arange(n))
    a, b = on.epoch_permutation(1, 1000), on.epoch_permutation(2, 1000)
    assert not np.array_equal(a, b) and np.array_equal(a, on.epoch_permutation(1, 1000))
    assert (a != np.arange(1000)).mean() > 0.9          # far from the identity
