"""Device-resident dataset + fused gather/normalise/flatten/one-hot kernel against the
numpy restatement of the README transform and of `iter_array` (bit-exact: u8 -> f64
conversion, one subtraction and one correctly rounded division per element)."""
import numpy as np
import pytest

import rstorch_b200 as rt
from oracle import oracle_np as on
from rstorch_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def test_gather_matches_the_readme_transform(ctx):
    images, labels = synth.mnist_like_u8(0, 0, 300)
    images[7] = 0                 # constant samples: (v - min) / 0 = NaN in the reference
    images[8] = 200
    images[9, 0, 0], images[9, 27, 27] = 3, 250          # min and max away from 0 and 255
    ds = rt.DeviceDataset(ctx, images, labels, 10)
    assert len(ds) == 300 and ds.features == 784
    rng = np.random.default_rng(0)
    for idx in (np.arange(32), np.array([9, 8, 7, 299, 0, 7]), rng.permutation(300)[:256]):
        X, T = ctx.empty(len(idx), 784), ctx.empty(len(idx), 10)
        ds.gather(idx, X, T)
        want_x, want_t = on.iter_array_batch(images, labels, idx, 10)
        assert np.array_equal(X.numpy(), want_x, equal_nan=True)
        assert np.array_equal(T.numpy(), want_t)
    assert np.isnan(want_x[:, 0]).sum() >= 1
    ds.close()


def test_data_loader_over_a_device_dataset(ctx):
    images, labels = synth.mnist_like_u8(1, 0, 100, side=4, classes=7)
    ds = rt.DeviceDataset(ctx, images, labels, 7)
    dl = rt.DataLoader(ds, 32, False, rt.SequentialSampler(len(ds)), ctx)
    assert len(dl) == 3
    got = [(x.numpy(), t.numpy()) for x, t in dl.iter_array()]
    assert len(got) == 3                                 # the 4 left-over samples are dropped
    for k, (x, t) in enumerate(got):
        want_x, want_t = on.iter_array_batch(images, labels, np.arange(k * 32, k * 32 + 32), 7)
        assert np.array_equal(x, want_x, equal_nan=True) and np.array_equal(t, want_t)
    # seeded shuffle: every epoch is a new permutation, every sample at most once per epoch
    dl2 = rt.DataLoader(ds, 25, True, rt.SequentialSampler(len(ds)), ctx, shuffle_seed=3)
    e1 = np.concatenate([t.numpy().argmax(axis=1) for _, t in dl2.iter_array()])
    e2 = np.concatenate([t.numpy().argmax(axis=1) for _, t in dl2.iter_array()])
    assert len(e1) == 100 and sorted(e1) == sorted(labels.tolist()) and not np.array_equal(e1, e2)


def test_training_from_the_device_dataset_matches_the_host_path(ctx):
    """Same samples through both loaders give the same training trajectory."""
    images, labels = synth.mnist_like_u8(2, 0, 128)
    X, T = on.iter_array_batch(images, labels, np.arange(128), 10)

    def run(loader):
        layers = []
        for l, (w, b) in enumerate(synth.mlp_weights(0, [784, 32, 10])):
            class Init(rt.InitParameters):
                def weight(self, i, o, w=w):
                    return w

                def bias(self, i, o, b=b):
                    return b
            layers.append(rt.Linear.new_with_kernel(w.shape[1], w.shape[0], Init(), ctx))
            if l == 0:
                layers.append(rt.ReLU())
        model, loss_fn, opt = rt.sequential(*layers), rt.CrossEntropyLoss(), rt.SGD.new(0.1)
        losses = []
        for x, t in loader.iter_array():
            losses.append(loss_fn.forward(model.forward(x), t))
            model.backward(loss_fn.backward(), need_input_grad=False)
            opt.step(model)
        return losses, [p.parm.numpy() for p in model.parameters()]

    dev = rt.DataLoader(rt.DeviceDataset(ctx, images, labels, 10), 32, False, rt.SequentialSampler(128), ctx)
    host = rt.DataLoader(rt.ArrayDataset(X, T), 32, False, rt.SequentialSampler(128), ctx)
    l1, p1 = run(dev)
    l2, p2 = run(host)
    assert l1 == l2 and len(l1) == 4
    for a, b in zip(p1, p2):
        assert np.array_equal(a, b)


def test_dataset_errors(ctx):
    images, labels = synth.mnist_like_u8(0, 0, 10, side=2)
    with pytest.raises(rt.RstError) as e:
        rt.DeviceDataset(ctx, images, labels, 5)          # labels reach 9: one_hot(9, 5) panics in the reference
    assert e.value.status == _lib.RST_ERR_INVALID_ARG
    ds = rt.DeviceDataset(ctx, images, labels, 10)
    X, T = ctx.empty(2, 4), ctx.empty(2, 10)
    with pytest.raises(rt.RstError) as e:
        ds.gather(np.array([0, 10]), X, T)                # index 10 is outside the 10 samples
    assert e.value.status == _lib.RST_ERR_INVALID_ARG
    with pytest.raises(rt.RstError) as e:
        ds.gather(np.array([0, 1, 2]), X, T)
    assert e.value.status == _lib.RST_ERR_SHAPE


def test_idx_files_to_device_batches(ctx, tmp_path):
    """The README's input path end to end: IDX files on disk -> MNIST dataset -> HBM ->
    `iter_array` batches of flatten(normalize_zero_one(x)) and one_hot(y, 10)."""
    import struct

    from rstorch_b200 import mnist
    images, labels = synth.mnist_like_u8(5, 0, 96)
    for name, arr in (("train-images-idx3-ubyte", images), ("train-labels-idx1-ubyte", labels)):
        with open(tmp_path / name, "wb") as f:
            f.write(struct.pack(">I", 8 * 256 + arr.ndim))
            f.write(struct.pack(f">{arr.ndim}I", *arr.shape))
            f.write(arr.tobytes())
    train = mnist.MNIST(str(tmp_path), train=True)
    loader = rt.DataLoader(train.to_device(ctx), 32, False, rt.SequentialSampler(len(train)), ctx)
    for k, (x, t) in enumerate(loader.iter_array()):
        want_x, want_t = on.iter_array_batch(images, labels, np.arange(k * 32, k * 32 + 32), 10)
        assert np.array_equal(x.numpy(), want_x) and np.array_equal(t.numpy(), want_t)
    assert k == 2


def test_staged_gather_eager_and_replayed(ctx):
    """The caller-filled index stage: same batches as `gather`, and a captured graph picks
    up the indices that are in the stage when it is replayed."""
    images, labels = synth.mnist_like_u8(4, 0, 200, side=6, classes=5)
    ds = rt.DeviceDataset(ctx, images, labels, 5)
    X, T = ctx.empty(48, 36), ctx.empty(48, 5)
    stage = ds.index_stage(48)
    assert stage.dtype == np.int64 and stage.shape == (48,)
    rng = np.random.default_rng(1)
    idx = rng.permutation(200)[:48]
    stage[:] = idx
    ds.gather_staged(48, X, T)
    want_x, want_t = on.iter_array_batch(images, labels, idx, 5)
    assert np.array_equal(X.numpy(), want_x, equal_nan=True) and np.array_equal(T.numpy(), want_t)
    assert ds.index_stage(48).ctypes.data == stage.ctypes.data          # the same buffer until it must grow

    with ctx.capture() as cap:
        ds.gather_staged(48, X, T)
    for seed in (2, 3, 4):
        idx = np.random.default_rng(seed).integers(0, 200, size=48)
        stage[:] = idx
        cap.graph.launch()
        want_x, want_t = on.iter_array_batch(images, labels, idx, 5)
        assert np.array_equal(X.numpy(), want_x, equal_nan=True) and np.array_equal(T.numpy(), want_t)
    ctx.check_device()

    # an index outside the dataset cannot be seen on the host: the kernel flags it
    stage[:] = np.arange(48)
    stage[5] = 200
    cap.graph.launch()
    with pytest.raises(rt.RstError) as e:
        ctx.check_device()
    assert e.value.status == _lib.RST_ERR_INVALID_ARG and "batch row 5" in str(e.value)
    x = X.numpy()
    assert np.isnan(x[5]).all() and np.array_equal(T.numpy()[5], np.zeros(5))
    assert np.array_equal(x[6], on.iter_array_batch(images, labels, np.array([6]), 5)[0][0], equal_nan=True)
    ctx.check_device()                                                   # the flag was cleared

    # shape and capacity errors
    with pytest.raises(rt.RstError) as e:
        ds.gather_staged(64, ctx.empty(64, 36), ctx.empty(64, 5))
    assert e.value.status == _lib.RST_ERR_STATE
    with pytest.raises(rt.RstError) as e:
        ds.gather_staged(48, ctx.empty(48, 35), T)
    assert e.value.status == _lib.RST_ERR_SHAPE
    ds.close()


def test_epoch_order_is_drawn_on_the_device_and_matches_the_host_mirror(ctx):
    """`Shuffler::shuffle` on the device (shuffler.rs:22-25): the kernel's permutation is
    compared bit for bit with its host mirror, and batches gathered through it with the
    README transform of the mirrored indices."""
    images, labels = synth.mnist_like_u8(5, 0, 1000, side=5, classes=6)
    ds = rt.DeviceDataset(ctx, images, labels, 6)
    assert np.array_equal(ds.epoch_order(), np.arange(1000))          # never shuffled: sampler order
    X, T = ctx.empty(64, 25), ctx.empty(64, 6)
    with pytest.raises(rt.RstError) as e:
        ds.gather_epoch(0, 64, X, T)
    assert e.value.status == _lib.RST_ERR_STATE
    for seed in (0, 1, 0xFFFFFFFFFFFFFFFF):
        ds.shuffle(seed)
        want = on.epoch_permutation(seed, 1000)
        assert np.array_equal(ds.epoch_order(), want)
        for first in (0, 64, 936):
            ds.gather_epoch(first, 64, X, T)
            want_x, want_t = on.iter_array_batch(images, labels, want[first:first + 64], 6)
            assert np.array_equal(X.numpy(), want_x, equal_nan=True) and np.array_equal(T.numpy(), want_t)
    with pytest.raises(rt.RstError) as e:
        ds.gather_epoch(960, 64, X, T)                                # runs past the dataset: the epoch ends
    assert e.value.status == _lib.RST_ERR_INVALID_ARG
    # sizes around the powers of four that change the Feistel width
    for n in (1, 2, 5, 16, 17, 255, 257):
        small = rt.DeviceDataset(ctx, images[:n], labels[:n], 6)
        small.shuffle(9)
        assert np.array_equal(small.epoch_order(), on.epoch_permutation(9, n))
        small.close()
    ctx.check_device()
    ds.close()


def test_shuffled_loader_over_a_device_dataset_keeps_the_order_on_the_device(ctx):
    images, labels = synth.mnist_like_u8(6, 0, 200, side=4, classes=5)
    ds = rt.DeviceDataset(ctx, images, labels, 5)
    dl = rt.DataLoader(ds, 32, True, rt.SequentialSampler(len(ds)), ctx, shuffle_seed=4)
    for epoch in range(2):
        got = [(x.numpy(), t.numpy()) for x, t in dl.iter_array()]
        assert len(got) == 6                                          # 8 left-over samples are dropped
        order = on.epoch_permutation(synth.stream_key(4, "shuffle", epoch), 200)
        for k, (x, t) in enumerate(got):
            want_x, want_t = on.iter_array_batch(images, labels, order[k * 32:(k + 1) * 32], 5)
            assert np.array_equal(x, want_x, equal_nan=True) and np.array_equal(t, want_t)
    ds.close()


def test_epoch_ends_at_the_first_missing_sample(ctx):
    """`dataset.get(index)?` (data_loader.rs:197): a sampler index outside the dataset ends
    the epoch there; indices after it are never used."""
    class Skipping:
        size = 12

        def iter(self):
            return iter([0, 1, 2, 3, 4, 5, 99, 6, 7, 8, 9, 10])

    X = np.arange(40, dtype=np.float64).reshape(10, 4)
    T = np.eye(10)
    dl = rt.DataLoader(rt.ArrayDataset(X, T), 2, False, Skipping(), ctx)
    got = [x.numpy() for x, _ in dl.iter_array()]
    assert len(got) == 3 and np.array_equal(np.concatenate(got), X[:6])
    dl.close()


def test_prefetching_loader_yields_the_same_batches(ctx):
    rng = np.random.default_rng(0)
    X, T = rng.standard_normal((230, 12)), rng.standard_normal((230, 3))
    ds = rt.ArrayDataset(X, T)
    for slots in (2, 3, 4):
        plain = rt.DataLoader(ds, 16, True, rt.SequentialSampler(len(ds)), ctx, slots=slots, shuffle_seed=1)
        ahead = rt.DataLoader(ds, 16, True, rt.SequentialSampler(len(ds)), ctx, slots=slots, shuffle_seed=1,
                              prefetch=True)
        a = [(x.numpy(), t.numpy()) for x, t in plain.iter_array()]
        b = [(x.numpy(), t.numpy()) for x, t in ahead.iter_array()]
        assert len(a) == len(b) == 14
        for (xa, ta), (xb, tb) in zip(a, b):
            assert np.array_equal(xa, xb) and np.array_equal(ta, tb)
        plain.close(); ahead.close()
