"""IDX (MNIST file format) reader and writer -- the on-disk format on the input side of the path.

The reference loads ``data/train-images.idx3-ubyte`` etc. through mnist.h:79-160: big-endian magic
2051 (images) / 2049 (labels), a big-endian count, for images two big-endian dimensions that must
be 28 x 28, then raw uint8 pixels / one label byte per item.  ``read_idx_pair`` mirrors that loader,
including its return codes; ``write_idx_pair`` produces files it (and therefore the unmodified
reference binary) accepts, which is how the synthetic sets are fed to the reference's own main().
"""
from __future__ import annotations

import os
import struct

import numpy as np

IMAGE_MAGIC = 2051
LABEL_MAGIC = 2049


def write_idx_pair(image_path: str, label_path: str, pixels_u8: np.ndarray, labels: np.ndarray) -> None:
    pixels_u8 = np.ascontiguousarray(pixels_u8, dtype=np.uint8)
    labels = np.ascontiguousarray(labels).astype(np.uint8)
    if pixels_u8.ndim != 3 or pixels_u8.shape[1:] != (28, 28):
        raise ValueError("pixels must be [n, 28, 28] uint8")
    if labels.shape != (pixels_u8.shape[0],):
        raise ValueError("one label per image")
    with open(image_path, "wb") as f:
        f.write(struct.pack(">IIII", IMAGE_MAGIC, pixels_u8.shape[0], 28, 28))
        f.write(pixels_u8.tobytes())
    with open(label_path, "wb") as f:
        f.write(struct.pack(">II", LABEL_MAGIC, labels.shape[0]))
        f.write(labels.tobytes())


def read_idx_pair(image_path: str, label_path: str):
    """Returns (code, pixels_u8 [n,28,28] | None, labels uint32 [n] | None) with mnist_load's codes:
    0 ok, -1 missing file, -2 bad image file, -3 bad label file, -4 count mismatch."""
    if not (os.path.exists(image_path) and os.path.exists(label_path)):
        return -1, None, None
    with open(image_path, "rb") as fi, open(label_path, "rb") as fl:
        head_i = fi.read(4)
        if len(head_i) < 4 or struct.unpack(">I", head_i)[0] != IMAGE_MAGIC:
            return -2, None, None
        head_l = fl.read(4)
        if len(head_l) < 4 or struct.unpack(">I", head_l)[0] != LABEL_MAGIC:
            return -3, None, None
        (n_img,) = struct.unpack(">I", fi.read(4))
        (n_lab,) = struct.unpack(">I", fl.read(4))
        if n_img != n_lab:
            return -4, None, None
        rows, cols = struct.unpack(">II", fi.read(8))
        if rows != 28 or cols != 28:
            return -2, None, None
        pixels = np.frombuffer(fi.read(n_img * 784), dtype=np.uint8)
        labels = np.frombuffer(fl.read(n_lab), dtype=np.uint8)
        if pixels.size != n_img * 784 or labels.size != n_lab:
            return -2, None, None
    return 0, pixels.reshape(n_img, 28, 28).copy(), labels.astype(np.uint32)


def write_reference_data_dir(directory: str, train, test) -> None:
    """Writes the four files the reference's loaddata() opens (main.cu:30-33) under directory/data/.
    ``train`` and ``test`` are (pixels_u8, labels) pairs."""
    d = os.path.join(directory, "data")
    os.makedirs(d, exist_ok=True)
    write_idx_pair(os.path.join(d, "train-images.idx3-ubyte"), os.path.join(d, "train-labels.idx1-ubyte"), *train)
    write_idx_pair(os.path.join(d, "t10k-images.idx3-ubyte"), os.path.join(d, "t10k-labels.idx1-ubyte"), *test)
