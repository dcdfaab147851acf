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


def test_initialisers_follow_their_distributions():
    w = rt.XavierNormal(seed=1).weight(300, 200)
    assert w.shape == (200, 300) and abs(w.std() / np.sqrt(2.0 / 500.0) - 1.0) < 0.02 and abs(w.mean()) < 0.01
    n = rt.Normal.new(2.0, 0.5, seed=1)
    v = n.weight(400, 100)
    assert v.shape == (100, 400) and abs(v.mean() - 2.0) < 0.01 and abs(v.std() - 0.5) < 0.01
    assert rt.Normal.new(0.0, float("nan")) is None and rt.Normal.new_std(float("inf")) is None
    assert np.array_equal(n.bias(400, 100), np.zeros((1, 100)))


def _write_idx(path, array, type_code):
    import struct
    with open(path, "wb") as f:
        f.write(struct.pack(">I", type_code * 256 + array.ndim))
        f.write(struct.pack(f">{array.ndim}I", *array.shape))
        f.write(array.astype(array.dtype.newbyteorder(">")).tobytes())


def test_idx_reader_and_mnist_dataset(tmp_path):
    from rstorch_b200 import mnist
    images, labels = synth.mnist_like_u8(4, 0, 50)
    _write_idx(tmp_path / "train-images-idx3-ubyte", images, 8)
    _write_idx(tmp_path / "train-labels-idx1-ubyte", labels, 8)
    ds = mnist.MNIST(str(tmp_path), train=True)
    assert len(ds) == 50 and np.array_equal(ds.data, images) and np.array_equal(ds.labels, labels)
    img, lab = ds.get(7)
    assert img.shape == (28, 28) and img.dtype == np.uint8 and lab == labels[7] and ds.get(50) is None
    with pytest.raises(FileNotFoundError):
        mnist.MNIST(str(tmp_path), train=False)                       # the t10k files are not there
    # big-endian multi-byte element types of the format (mnist.rs:258-263)
    vals = np.array([[1, -2, 300], [-40000, 5, 6]], dtype=np.int32)
    _write_idx(tmp_path / "i32", vals, 12)
    assert np.array_equal(mnist.read_sn3(str(tmp_path / "i32")), vals)
    f64 = np.array([1.5, -2.25, 1e300])
    _write_idx(tmp_path / "f64", f64, 14)
    assert np.array_equal(mnist.read_sn3(str(tmp_path / "f64"), ndim=1, type_code=14), f64)
    # the reference asserts on the header (mnist.rs:284-285) and unwraps the reshape
    with pytest.raises(ValueError):
        mnist.read_image_file(str(tmp_path / "train-labels-idx1-ubyte"))
    with pytest.raises(ValueError):
        mnist.read_sn3(str(tmp_path / "i32"), type_code=8)
    with open(tmp_path / "short", "wb") as f:
        f.write(open(tmp_path / "train-images-idx3-ubyte", "rb").read()[:1000])
    with pytest.raises(ValueError):
        mnist.read_image_file(str(tmp_path / "short"))


def test_default_initialiser_gives_every_layer_its_own_stream():
    """The reference draws every layer from the thread generator (he.rs:13): layers built
    without an initialiser must not share weights, whatever their shapes."""
    from rstorch_b200 import module
    module.reset_default_init(0)
    a, b = rt.Linear(100, 100), rt.Linear(100, 100)
    assert not np.array_equal(a._host_weight, b._host_weight)
    c, d = rt.Linear(784, 100), rt.Linear(100, 10)
    # the underlying unit normals (weights rescaled by sqrt(fan-in)) share no prefix either
    zc, zd = c._host_weight.reshape(-1) * np.sqrt(784.0), d._host_weight.reshape(-1) * np.sqrt(100.0)
    assert not np.allclose(zc[:1000], zd[:1000])
    # a model built in order in a fresh process reproduces the benchmark's seed-0 weights
    module.reset_default_init(0)
    dims = [784, 100, 100, 10]
    layers = [rt.Linear(dims[l], dims[l + 1]) for l in range(3)]
    for lin, (w, bias) in zip(layers, synth.mlp_weights(0, dims)):
        assert np.array_equal(lin._host_weight, w) and np.array_equal(lin._host_bias, bias)


def test_linear_without_bias_has_one_parameter_pair():
    lin = rt.Linear.without_bias(4, 3)
    assert lin._host_bias is None and not lin.has_bias and lin._host_weight.shape == (3, 4)
    with pytest.raises(RuntimeError, match="before any backward"):
        lin.parameters()


def test_basic_model_follows_the_reference_step_order():
    """model.rs:19-31 with stand-in parts: forward, loss.forward, loss.backward, backward, step."""
    calls = []

    class M(rt.Module):
        def forward(self, x):
            calls.append("module.forward"); return x

        def backward(self, g):
            calls.append("module.backward"); return g

    class L(rt.Loss):
        def forward(self, p, t):
            calls.append("loss.forward"); return 0.0

        def backward(self):
            calls.append("loss.backward"); return None

    class O(rt.Optimizer):
        def step(self, module):
            calls.append("optim.step")

    model = rt.BasicModel.new(M(), L(), O())
    model.step("x", "t")
    assert calls == ["module.forward", "loss.forward", "loss.backward", "module.backward", "optim.step"]
    assert model.predict("x") == "x" and calls[-1] == "module.forward"
