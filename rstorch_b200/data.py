"""Batch assembly: `DataLoader::iter_array` (src/data/data_loader.rs:42-93,180-208)
with the batches staged through pinned host memory and a copy stream."""
from __future__ import annotations

import ctypes as C
from typing import Iterator

import numpy as np

from .core import Context, Tensor


class ArrayDataset:
    """Random-access dataset of (sample, target) rows held as two host arrays;
    `get`/`len` follow the `Dataset` trait (src/data/dataset/mod.rs:15-57)."""

    def __init__(self, samples: np.ndarray, targets: np.ndarray):
        if len(samples) != len(targets):
            raise ValueError("samples and targets differ in length")
        self.samples = np.asarray(samples, dtype=np.float64).reshape(len(samples), -1)
        self.targets = np.asarray(targets, dtype=np.float64).reshape(len(targets), -1)

    def get(self, index: int):
        if not 0 <= index < len(self.samples):
            return None
        return self.samples[index], self.targets[index]

    def __len__(self) -> int:
        return len(self.samples)


class DeviceDataset:
    """u8 samples and labels resident in HBM (the item type of the reference's MNIST
    dataset, src/data/dataset/hub/mnist.rs:181-194) with the README transform
    `(flatten(normalize_zero_one(x)), one_hot(y, classes))` (README.md:44) applied by
    the gather kernel when a batch is built."""

    def __init__(self, ctx: Context, images: np.ndarray, labels: np.ndarray, classes: int):
        images = np.ascontiguousarray(images, dtype=np.uint8)
        labels = np.ascontiguousarray(labels, dtype=np.uint8).reshape(-1)
        if len(images) != len(labels):
            raise ValueError("images and labels differ in length")
        self.ctx, self.n, self.classes = ctx, len(labels), int(classes)
        self.features = int(np.prod(images.shape[1:])) if images.ndim > 1 else 1
        h = C.c_void_p()
        ctx._check(ctx._lib.rst_dataset_create_u8(ctx.handle, images.ctypes.data_as(C.c_void_p),
                                                  labels.ctypes.data_as(C.c_void_p), self.n, self.features,
                                                  self.classes, C.byref(h)))
        self.handle = h

    def __len__(self) -> int:
        return self.n

    def gather(self, indices: np.ndarray, X: Tensor, T: Tensor) -> None:
        idx = np.ascontiguousarray(indices, dtype=np.int64)
        self.ctx._check(self.ctx._lib.rst_dataset_gather(self.handle, idx.ctypes.data_as(C.POINTER(C.c_int64)),
                                                         len(idx), X.handle, T.handle))

    def index_stage(self, batch: int) -> np.ndarray:
        """The dataset's pinned index buffer as an int64 array of `batch` entries; write the
        sample indices of the next batch into it and call `gather_staged`."""
        p = C.POINTER(C.c_int64)()
        self.ctx._check(self.ctx._lib.rst_dataset_index_stage(self.handle, int(batch), C.byref(p)))
        return np.ctypeslib.as_array(p, shape=(int(batch),))

    def gather_staged(self, batch: int, X: Tensor, T: Tensor) -> None:
        """Builds the batch of the indices currently in the index stage.  May be captured
        into a graph; each replay uses the indices the stage holds at that moment."""
        self.ctx._check(self.ctx._lib.rst_dataset_gather_staged(self.handle, int(batch), X.handle, T.handle))

    def shuffle(self, seed: int) -> None:
        """Draws the order of the next epoch on the device (`Shuffler::shuffle`,
        src/data/dataset/shuffler.rs:22-25): a keyed bijection of [0, len)."""
        self.ctx._check(self.ctx._lib.rst_dataset_shuffle(self.handle, int(seed) & 0xFFFFFFFFFFFFFFFF))

    def epoch_order(self) -> np.ndarray:
        """The current epoch's order of the samples (identity before the first shuffle)."""
        out = np.empty(self.n, dtype=np.int64)
        self.ctx._check(self.ctx._lib.rst_dataset_epoch_order(self.handle, out.ctypes.data_as(C.POINTER(C.c_int64))))
        return out

    def gather_epoch(self, first: int, batch: int, X: Tensor, T: Tensor) -> None:
        """Builds the batch of epoch positions [first, first + batch) (`Shuffler::get`,
        shuffler.rs:31-33); no sample index leaves the device."""
        self.ctx._check(self.ctx._lib.rst_dataset_gather_epoch(self.handle, int(first), int(batch), X.handle, T.handle))

    def close(self) -> None:
        if self.handle is not None and self.handle.value and self.ctx.handle.value:
            self.ctx._lib.rst_dataset_destroy(self.handle)
        self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class SequentialSampler:
    """0..size (src/data/sampler.rs:31-43)."""

    def __init__(self, size: int):
        self.size = int(size)

    def iter(self) -> Iterator[int]:
        return iter(range(self.size))


class DataLoader:
    """`DataLoader::new(dataset, batch_size, shuffle, sampler)`.

    `iter_array` yields `(X, T)` device tensors of `batch_size` consecutive sampler
    indices and, like the reference, ends the epoch at the first batch it cannot
    fill (the remainder is dropped, data_loader.rs:69-71,197).  The reference's
    shuffle draws from an unseedable thread RNG (dataset/shuffler.rs:15-25); here
    it is a permutation from `shuffle_seed`, redrawn at every `iter_array` call
    (data_loader.rs:88-92).  Over a `DeviceDataset` the permutation is drawn by a
    kernel and stays on the device: epoch e uses the key `synth.stream_key(
    shuffle_seed, "shuffle", e)`."""

    def __init__(self, dataset: ArrayDataset, batch_size: int, shuffle: bool, sampler: SequentialSampler,
                 ctx: Context, slots: int = 2, shuffle_seed: int = 0, prefetch: bool = False):
        """`prefetch=True` assembles batches on a helper thread: while the GPU runs step k
        the thread gathers the rows of batch k+2 into a pinned slot and the copy stream
        moves batch k+1 to the device (use three slots to keep all three in flight)."""
        self.dataset, self.batch_size, self.sampler, self.ctx = dataset, int(batch_size), sampler, ctx
        self._prefetch = bool(prefetch)
        self._shuffle = bool(shuffle)
        self._shuffle_seed, self._epoch = int(shuffle_seed), 0
        self._rng = np.random.default_rng(shuffle_seed)
        self._slots = int(slots)
        self._stager = None
        self._views: dict = {}            # slot -> pinned host arrays
        self._device_pairs: dict = {}     # slot -> wrappers of the slot's device tensors

    def __len__(self) -> int:
        return len(self.dataset) // self.batch_size

    def is_empty(self) -> bool:
        return len(self.dataset) < self.batch_size

    # -- staging -------------------------------------------------------------
    def _ensure_stager(self):
        if self._stager is None:
            h = C.c_void_p()
            lib, ctx = self.ctx._lib, self.ctx
            ctx._check(lib.rst_stager_create(ctx.handle, self.batch_size, self.dataset.samples.shape[1],
                                             self.dataset.targets.shape[1], self._slots, C.byref(h)))
            self._stager = h
        return self._stager

    def _host_views(self, slot: int):
        """The pinned arrays of a slot, once the previous copy out of them has finished.  The
        arrays are made once per slot (the addresses never change); every call still goes
        through rst_stager_host, which is what waits for that copy."""
        lib, ctx = self.ctx._lib, self.ctx
        views = self._views.get(slot)
        if views is not None:
            ctx._check(lib.rst_stager_host(self._stager, slot, None, None))
            return views
        px, pt = C.POINTER(C.c_double)(), C.POINTER(C.c_double)()
        ctx._check(lib.rst_stager_host(self._stager, slot, C.byref(px), C.byref(pt)))
        b = self.batch_size
        x = np.ctypeslib.as_array(px, shape=(b, self.dataset.samples.shape[1]))
        t = np.ctypeslib.as_array(pt, shape=(b, self.dataset.targets.shape[1]))
        self._views[slot] = (x, t)
        return x, t

    def _assemble(self, views, indices: np.ndarray) -> None:
        """`ArrayDataLoaderIter::next` (data_loader.rs:192-207): the rows of the batch's
        samples, one after the other, into the two batch arrays.  The indices were checked
        against the dataset when the epoch's order was made, so `clip` never alters one; it
        only spares numpy's bounds-checking mode its temporary copy of the output."""
        x, t = views
        np.take(self.dataset.samples, indices, axis=0, out=x, mode="clip")
        np.take(self.dataset.targets, indices, axis=0, out=t, mode="clip")

    def _fill(self, slot: int, indices: np.ndarray) -> None:
        self._assemble(self._host_views(slot), indices)
        self.ctx._check(self.ctx._lib.rst_stager_submit(self._stager, slot))

    def _iter_prefetched(self, order: np.ndarray) -> Iterator[tuple[Tensor, Tensor]]:
        """While the caller works on batch k, the copy stream moves batch k+1 to the device and
        helper threads gather the rows of batches k+2 .. k+slots-1 into their pinned slots
        (one thread per batch; numpy's `take` runs without the interpreter lock).  Only the main
        thread calls the library; the helpers touch the pinned host arrays alone.  With two
        slots nothing can be assembled ahead and the batches are built one by one."""
        import concurrent.futures as cf
        b, S, lib = self.batch_size, self._slots, self.ctx._lib
        n_batches = len(order) // b
        if n_batches == 0:
            return
        with cf.ThreadPoolExecutor(max_workers=max(1, S - 2)) as pool:
            pending: dict[int, cf.Future] = {}
            started = 0

            def start_up_to(last: int) -> None:
                # rst_stager_host waits until the previous copy out of that pinned slot is done;
                # batch j reuses the slot of batch j - S, whose copy was queued S - 1 batches ago
                nonlocal started
                while started <= min(last, n_batches - 1):
                    pending[started] = pool.submit(self._assemble, self._host_views(started % S),
                                                   order[started * b:(started + 1) * b])
                    started += 1

            start_up_to(max(1, S - 2))
            pending.pop(0).result()
            self.ctx._check(lib.rst_stager_submit(self._stager, 0))
            for k in range(n_batches):
                if k + 1 < n_batches:
                    start_up_to(k + 1)                   # only needed when fewer than three slots
                    pending.pop(k + 1).result()
                    self.ctx._check(lib.rst_stager_submit(self._stager, (k + 1) % S))
                if S >= 3:
                    start_up_to(k + S - 1)
                yield self._acquire(k % S)

    def _acquire(self, slot: int) -> tuple[Tensor, Tensor]:
        lib, ctx = self.ctx._lib, self.ctx
        hx, ht = C.c_void_p(), C.c_void_p()
        ctx._check(lib.rst_stager_acquire(self._stager, slot, C.byref(hx), C.byref(ht)))
        pair = self._device_pairs.get(slot)
        if pair is None or pair[0].handle.value != hx.value:
            b = self.batch_size
            # the stager owns these tensors; the wrappers must not free them
            pair = (Tensor(ctx, hx, b, self.dataset.samples.shape[1], owns=False),
                    Tensor(ctx, ht, b, self.dataset.targets.shape[1], owns=False))
            self._device_pairs[slot] = pair
        return pair

    def _iter_device(self, order: np.ndarray) -> Iterator[tuple[Tensor, Tensor]]:
        """Batches of a DeviceDataset: the gather kernel writes into a small ring of
        output tensors (a batch stays valid until `slots` later batches were asked for)."""
        ds, b = self.dataset, self.batch_size
        ring = max(2, self._slots)
        if getattr(self, "_out_ring", None) is None or len(self._out_ring) != ring:
            self._out_ring = [(self.ctx.empty(b, ds.features), self.ctx.empty(b, ds.classes)) for _ in range(ring)]
        for k in range(len(order) // b):
            X, T = self._out_ring[k % ring]
            ds.gather(order[k * b:(k + 1) * b], X, T)
            yield X, T

    def _iter_device_shuffled(self) -> Iterator[tuple[Tensor, Tensor]]:
        """Epoch of a shuffled DeviceDataset under the sequential sampler: the order is drawn
        and consumed on the device."""
        from . import synth
        ds, b = self.dataset, self.batch_size
        ds.shuffle(synth.stream_key(self._shuffle_seed, "shuffle", self._epoch))
        self._epoch += 1
        ring = max(2, self._slots)
        if getattr(self, "_out_ring", None) is None or len(self._out_ring) != ring:
            self._out_ring = [(self.ctx.empty(b, ds.features), self.ctx.empty(b, ds.classes)) for _ in range(ring)]
        for k in range(min(self.sampler.size, len(ds)) // b):
            X, T = self._out_ring[k % ring]
            ds.gather_epoch(k * b, b, X, T)
            yield X, T

    def iter_array(self) -> Iterator[tuple[Tensor, Tensor]]:
        if self._shuffle and isinstance(self.dataset, DeviceDataset) and isinstance(self.sampler, SequentialSampler):
            yield from self._iter_device_shuffled()
            return
        order = np.fromiter(self.sampler.iter(), dtype=np.int64)
        # `dataset.get(index)?` returns None at the first index the dataset does not hold and
        # that ends the epoch (data_loader.rs:197): later indices are never looked at
        missing = np.flatnonzero((order < 0) | (order >= len(self.dataset)))
        if missing.size:
            order = order[:missing[0]]
        if self._shuffle:
            perm = self._rng.permutation(len(self.dataset))
            order = perm[order]
        if isinstance(self.dataset, DeviceDataset):
            yield from self._iter_device(order)
            return
        self._ensure_stager()
        if self._prefetch and self._slots >= 2:
            yield from self._iter_prefetched(order)
            return
        n_batches = len(order) // self.batch_size
        b = self.batch_size
        # keep `slots - 1` batches in flight ahead of the one being consumed
        ahead = min(self._slots - 1, n_batches) if self._slots > 1 else 0
        for k in range(ahead):
            self._fill(k % self._slots, order[k * b:(k + 1) * b])
        for k in range(n_batches):
            slot = k % self._slots
            if self._slots == 1:
                self._fill(slot, order[k * b:(k + 1) * b])
            yield self._acquire(slot)
            nxt = k + ahead
            if self._slots > 1 and nxt < n_batches:
                # the slot consumed one iteration ago is free again
                self._fill(nxt % self._slots, order[nxt * b:(nxt + 1) * b])

    def close(self) -> None:
        if self._stager is not None and self.ctx.handle.value:
            self.ctx._lib.rst_stager_destroy(self._stager)
        self._stager = None
        self._views, self._device_pairs = {}, {}

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
