"""Reader of the IDX ("sn3") files the reference's MNIST dataset parses
(src/data/dataset/hub/mnist.rs:241-313) and the dataset object built on them.

File layout (all integers big-endian): a 32-bit magic whose low byte is the number
of dimensions and whose next byte is the element type (8 = u8, 9 = i8, 11 = i16,
12 = i32, 13 = f32, 14 = f64; mnist.rs:258-263), then one 32-bit extent per dimension,
then the elements in row-major order.  The reference downloads the four files over
HTTP (mnist.rs:98-161); this module reads files that are already on disk and never
touches the network.
"""
from __future__ import annotations

import os
import struct

import numpy as np

from .core import Context
from .data import DeviceDataset

_TYPES = {8: ">u1", 9: ">i1", 11: ">i2", 12: ">i4", 13: ">f4", 14: ">f8"}


def read_sn3(path: str, ndim: int | None = None, type_code: int | None = None) -> np.ndarray:
    """Parses one IDX file.  `ndim` / `type_code`, when given, must match the header,
    as the reference asserts (mnist.rs:284-285)."""
    with open(path, "rb") as f:
        raw = f.read()
    if len(raw) < 4:
        raise ValueError(f"{path}: too short for an IDX header")
    magic = struct.unpack(">I", raw[:4])[0]
    nd, ty = magic % 256, magic // 256
    if ndim is not None and nd != ndim:
        raise ValueError(f"{path}: {nd} dimensions, expected {ndim}")
    if type_code is not None and ty != type_code:
        raise ValueError(f"{path}: element type {ty}, expected {type_code}")
    if ty not in _TYPES:
        raise ValueError(f"{path}: unknown element type {ty}")
    if len(raw) < 4 + 4 * nd:
        raise ValueError(f"{path}: header truncated")
    shape = struct.unpack(f">{nd}I", raw[4:4 + 4 * nd])
    data = np.frombuffer(raw, dtype=_TYPES[ty], offset=4 + 4 * nd)
    if data.size != int(np.prod(shape, dtype=np.int64)):
        raise ValueError(f"{path}: {data.size} elements for shape {shape}")       # into_shape(...).unwrap()
    return data.astype(data.dtype.newbyteorder("=")).reshape(shape)


def read_image_file(path: str) -> np.ndarray:
    """(n, rows, cols) u8 (mnist.rs:310-313)."""
    return read_sn3(path, ndim=3, type_code=8)


def read_label_file(path: str) -> np.ndarray:
    """(n,) u8 (mnist.rs:305-308)."""
    return read_sn3(path, ndim=1, type_code=8)


class MNIST:
    """`MNIST::new(root, train, download)` over files already present in `root`
    (`train-images-idx3-ubyte`, `train-labels-idx1-ubyte`, `t10k-...`; mnist.rs:164-179).
    Items are `(28x28 u8 image, u8 label)` (mnist.rs:181-194)."""

    def __init__(self, root: str, train: bool = True, download: bool = False):
        start = "train" if train else "t10k"
        images = os.path.join(root, f"{start}-images-idx3-ubyte")
        labels = os.path.join(root, f"{start}-labels-idx1-ubyte")
        if not (os.path.exists(images) and os.path.exists(labels)):
            hint = " (downloading is not supported: place the decompressed IDX files there)" if download else ""
            raise FileNotFoundError(f"Dataset not found in {root}{hint}")            # assert! at mnist.rs:66-69
        self.data, self.labels = read_image_file(images), read_label_file(labels)
        if len(self.data) != len(self.labels):
            raise ValueError("image and label files differ in length")               # assert_eq! at mnist.rs:176

    def __len__(self) -> int:
        return len(self.labels)

    def get(self, index: int):
        if not 0 <= index < len(self):
            return None
        return self.data[index].copy(), self.labels[index].copy()

    def to_device(self, ctx: Context, classes: int = 10) -> DeviceDataset:
        """Places the samples in HBM; batches then come from the fused
        gather/normalise/flatten/one-hot kernel (README.md:44 transform)."""
        return DeviceDataset(ctx, self.data, self.labels, classes)
