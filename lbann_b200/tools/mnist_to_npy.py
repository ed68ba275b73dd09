"""MNIST idx files (optionally gzipped) to ``.npy`` and ``.npz`` for the numpy readers.

For each split: ``<split>_images.npy`` ([N, 784] uint8), ``<split>_labels.npy`` ([N] uint8),
``<split>.npy`` ([N, 785]: pixels then the label, the layout the ``numpy`` reader takes with
``has_labels``) and ``<split>.npz`` (arrays ``data`` and ``labels``, the ``numpy_npz``
reader's layout).  Counterpart of tools/mnist/mnist_to_npy_and_npz.py.
"""
from __future__ import annotations

import argparse
import gzip
import os
import struct

import numpy as np


def read_idx(path: str) -> np.ndarray:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rb") as f:
        zero, dtype_code, ndim = struct.unpack(">HBB", f.read(4))
        if zero != 0 or dtype_code != 0x08:
            raise ValueError(f"{path}: not an unsigned-byte idx file")
        shape = struct.unpack(">" + "I" * ndim, f.read(4 * ndim))
        data = np.frombuffer(f.read(), dtype=np.uint8)
    return data.reshape(shape)


def convert(images_path: str, labels_path: str, out_dir: str, split: str) -> dict:
    images = read_idx(images_path)
    labels = read_idx(labels_path)
    if images.shape[0] != labels.shape[0]:
        raise ValueError("images and labels differ in length")
    flat = images.reshape(images.shape[0], -1)
    os.makedirs(out_dir, exist_ok=True)
    out = {
        "images": os.path.join(out_dir, f"{split}_images.npy"),
        "labels": os.path.join(out_dir, f"{split}_labels.npy"),
        "combined": os.path.join(out_dir, f"{split}.npy"),
        "npz": os.path.join(out_dir, f"{split}.npz"),
    }
    np.save(out["images"], flat)
    np.save(out["labels"], labels)
    np.save(out["combined"], np.concatenate([flat, labels[:, None]], axis=1))
    np.savez(out["npz"], data=flat, labels=labels)
    return out


def _find(data_dir: str, stem: str) -> str:
    for name in (stem, stem + ".gz", stem.replace("-idx", ".idx"), stem.replace("-idx", ".idx") + ".gz"):
        p = os.path.join(data_dir, name)
        if os.path.exists(p):
            return p
    raise FileNotFoundError(f"{stem}[.gz] not found in {data_dir}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("data_dir", help="directory with the four idx files")
    ap.add_argument("out_dir")
    a = ap.parse_args(argv)
    for split, stem in (("train", "train"), ("test", "t10k")):
        out = convert(_find(a.data_dir, f"{stem}-images-idx3-ubyte"),
                      _find(a.data_dir, f"{stem}-labels-idx1-ubyte"), a.out_dir, split)
        print(f"{split}: {out['combined']} {out['npz']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
