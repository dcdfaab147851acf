"""Host-side logic that needs no device: synthetic streams, sharding, the editing
API of Sequential, the reference's panics mapped to exceptions."""
import numpy as np
import pytest

import rstorch_b200 as rt
from rstorch_b200 import synth


def test_streams_are_reproducible_and_sliceable():
    k = synth.stream_key(0, "x")
    a = synth.uniform(k, 1000)
    assert np.array_equal(a[100:200], synth.uniform(k, 100, offset=100))
    assert a.min() >= 0.0 and a.max() < 1.0
    n = synth.normal(k, 20000)
    assert abs(n.mean()) < 0.03 and abs(n.std() - 1.0) < 0.03
    assert np.array_equal(n[50:60], synth.normal(k, 10, offset=50))
    assert synth.stream_key(0, "x") != synth.stream_key(1, "x") != synth.stream_key(0, "y")


def test_mnist_like_distribution():
    X, T = synth.mnist_like(0, 0, 512)
    assert X.shape == (512, 784) and T.shape == (512, 10)
    zero = (X == 0.0).mean()
    assert 0.80 < zero < 0.82
    nz = X[X != 0.0]
    assert nz.min() > 0.0 and nz.max() <= 1.0
    assert np.array_equal(T.sum(axis=1), np.ones(512)) and set(np.unique(T)) == {0.0, 1.0}
    X2, T2 = synth.mnist_like(0, 100, 28)
    assert np.array_equal(X2, X[100:128]) and np.array_equal(T2, T[100:128])


def test_gaussian_batch_shards_match_the_global_batch():
    Xg, Tg = synth.gaussian_batch(3, step=2, first_row=0, rows=64, features=12, classes=7, global_batch=64)
    for rank in range(4):
        first, rows = rt.shard_rows(64, rank, 4)
        Xr, Tr = synth.gaussian_batch(3, 2, first, rows, 12, 7, 64)
        assert np.array_equal(Xr, Xg[first:first + rows]) and np.array_equal(Tr, Tg[first:first + rows])
    with pytest.raises(ValueError):
        rt.shard_rows(65, 0, 4)


def test_weights_follow_the_reference_initialiser():
    (w, b), = synth.mlp_weights(0, [4096, 512])
    assert w.shape == (512, 4096) and b.shape == (1, 512) and not b.any()
    assert abs(w.std() * np.sqrt(4096) - 1.0) < 0.01          # sigma = 1/sqrt(in), he.rs:12
    k = rt.KaimingNormal(seed=0)
    assert np.array_equal(k.weight(4096, 512), w)              # same stream as the bench


def test_sgd_tensor_sizes():
    sizes = synth.sgd_tensor_sizes(0, 1 << 20, 64)
    assert len(sizes) == 64 and sum(sizes) == 1 << 20 and min(sizes) > 0


def test_sequential_editing_api():
    m = rt.sequential(rt.Identity(), rt.Linear(3, 4), rt.ReLU())
    assert len(m) == 3 and not m.is_empty()
    m.push(rt.Linear(4, 2))
    m.insert(0, rt.Identity())
    assert len(m) == 5 and isinstance(m.layers[0], rt.Identity)
    assert m.remove(99) is None                                # sequential.rs:43-48
    assert isinstance(m.remove(0), rt.Identity) and len(m) == 4
    assert rt.Sequential().is_empty()
    assert len(rt.sequential([rt.ReLU(), rt.ReLU()])) == 2


def test_calls_out_of_order_raise_like_the_reference_panics():
    lin = rt.Linear(3, 2)
    with pytest.raises(RuntimeError, match="without a preceding forward"):
        lin._backward(None, False, True)
    with pytest.raises(RuntimeError, match="before any backward"):
        lin.parameters()
    with pytest.raises(RuntimeError, match="without a preceding forward"):
        rt.ReLU().backward(None)
    with pytest.raises(RuntimeError, match="without a preceding forward"):
        rt.CrossEntropyLoss().backward()


def test_linear_holds_weight_out_by_in_and_bias_one_by_out():
    class Fixed(rt.InitParameters):
        def weight(self, i, o):
            return np.array([[1.0, 0.5]])

        def bias(self, i, o):
            return np.array([[10.0]])

    lin = rt.Linear.new_with_kernel(2, 1, Fixed())
    assert lin._host_weight.shape == (1, 2) and lin._host_bias.shape == (1, 1)
    assert rt.Linear(5, 3)._host_weight.shape == (3, 5)


def test_one_hot():
    assert rt.one_hot(3, 5).tolist() == [0, 0, 0, 1, 0]
    with pytest.raises(IndexError):
        rt.one_hot(5, 5)
