"""Mean image of an image list.

``compute``: every rank (``torch.distributed`` when initialised, else one process) reads its
stride of the list, centre-crops to ``--crop W H`` (after an optional resize of the shorter
side to ``--resize``), accumulates the per-pixel sum in float64; the sums are added over
the ranks and rank 0 writes ``mean.npy`` ([H, W, C] float32) and, with ``--save-cropped``,
the cropped images as ``.npy`` next to it.  ``uniform``: an image filled with given
per-channel values, or with the per-channel mean of an existing image.

The reference tool does the same with OpenCV and MPI (tools/compute_mean/compute_mean.cpp,
process_images.cpp, uniform_mean.cpp); images are read here with ``lbann_b200.data``'s
decoder (``.npy`` arrays and the formats PIL can read when it is installed).
"""
from __future__ import annotations

import argparse
import os
from typing import List, Optional, Sequence

import numpy as np


def _load(path: str) -> np.ndarray:
    if path.endswith(".npy"):
        img = np.load(path)
    else:
        try:
            from PIL import Image
        except ImportError as e:      # pragma: no cover - depends on the image
            raise RuntimeError(f"reading '{path}' needs PIL; .npy images need nothing") from e
        img = np.asarray(Image.open(path))
    if img.ndim == 2:
        img = img[:, :, None]
    return img


def _resize_shorter(img: np.ndarray, size: int) -> np.ndarray:
    """Nearest-neighbour resize that brings the shorter side to ``size``."""
    h, w = img.shape[:2]
    s = size / min(h, w)
    nh, nw = max(int(round(h * s)), size), max(int(round(w * s)), size)
    yi = np.minimum((np.arange(nh) / s).astype(np.int64), h - 1)
    xi = np.minimum((np.arange(nw) / s).astype(np.int64), w - 1)
    return img[yi][:, xi]


def centre_crop(img: np.ndarray, w: int, h: int) -> np.ndarray:
    ih, iw = img.shape[:2]
    if ih < h or iw < w:
        raise ValueError(f"image {iw}x{ih} is smaller than the crop {w}x{h}")
    y0, x0 = (ih - h) // 2, (iw - w) // 2
    return img[y0:y0 + h, x0:x0 + w]


def read_image_list(list_file: str) -> List[str]:
    out = []
    with open(list_file) as f:
        for line in f:
            line = line.strip()
            if line:
                out.append(line.split()[0])
    return out


def mean_image(root: str, names: Sequence[str], crop, resize: Optional[int] = None,
               save_dir: Optional[str] = None, rank: int = 0, world: int = 1,
               allreduce=None) -> Optional[np.ndarray]:
    """Per-pixel mean over ``names`` (relative to ``root``); collective over ``world`` ranks
    when ``allreduce(array) -> array`` is given.  Returns the mean on every rank."""
    w, h = crop
    total = None
    count = 0
    for i in range(rank, len(names), world):
        img = _load(os.path.join(root, names[i]))
        if resize:
            img = _resize_shorter(img, resize)
        img = centre_crop(img, w, h)
        if total is None:
            total = np.zeros(img.shape, dtype=np.float64)
        total += img
        count += 1
        if save_dir:
            dst = os.path.join(save_dir, os.path.splitext(names[i])[0] + ".npy")
            os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
            np.save(dst, img)
    packed = np.concatenate([(total if total is not None else np.zeros(0)).reshape(-1),
                             np.array([float(count)])])
    if allreduce is not None:
        shape = np.array(total.shape if total is not None else (0, 0, 0), dtype=np.float64)
        shape = allreduce(shape, "max")
        if total is None:
            packed = np.zeros(int(np.prod(shape)) + 1)
        packed = allreduce(packed, "sum")
        total_shape = tuple(int(s) for s in shape)
    else:
        total_shape = total.shape if total is not None else (0,)
    n = packed[-1]
    if n == 0:
        return None
    return (packed[:-1] / n).reshape(total_shape).astype(np.float32)


def uniform_image(w: int, h: int, values: Sequence[float]) -> np.ndarray:
    return np.broadcast_to(np.asarray(values, dtype=np.float32), (h, w, len(values))).copy()


def channel_mean(img: np.ndarray) -> np.ndarray:
    return img.reshape(-1, img.shape[-1]).mean(0)


def _dist_allreduce():
    try:
        import torch
        import torch.distributed as dist
    except ImportError:      # pragma: no cover
        return None, 0, 1
    if not (dist.is_available() and dist.is_initialized()):
        if "RANK" in os.environ and "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1:
            dist.init_process_group("gloo")
        else:
            return None, 0, 1

    def allreduce(a: np.ndarray, op: str) -> np.ndarray:
        t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float64))
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
        return t.numpy()
    return allreduce, dist.get_rank(), dist.get_world_size()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("compute", help="mean of an image list")
    c.add_argument("root")
    c.add_argument("list_file")
    c.add_argument("out_dir")
    c.add_argument("--crop", nargs=2, type=int, required=True, metavar=("W", "H"))
    c.add_argument("--resize", type=int, default=None, help="shorter side before the crop")
    c.add_argument("--save-cropped", action="store_true")
    u = sub.add_parser("uniform", help="an image filled with per-channel values")
    u.add_argument("out_file")
    u.add_argument("--size", nargs=2, type=int, metavar=("W", "H"))
    u.add_argument("--values", nargs="+", type=float)
    u.add_argument("--from-image")
    a = ap.parse_args(argv)
    if a.cmd == "uniform":
        if a.from_image:
            img = _load(a.from_image)
            vals = channel_mean(img)
            w, h = (a.size if a.size else (img.shape[1], img.shape[0]))
        else:
            if not (a.values and a.size):
                ap.error("uniform needs --values and --size, or --from-image")
            vals, (w, h) = a.values, a.size
        np.save(a.out_file, uniform_image(w, h, vals))
        print("per-channel values:", " ".join(f"{v:.4f}" for v in vals))
        return 0
    allreduce, rank, world = _dist_allreduce()
    names = read_image_list(a.list_file)
    os.makedirs(a.out_dir, exist_ok=True)
    mean = mean_image(a.root, names, tuple(a.crop), a.resize,
                      os.path.join(a.out_dir, "cropped") if a.save_cropped else None,
                      rank, world, allreduce)
    if rank == 0 and mean is not None:
        np.save(os.path.join(a.out_dir, "mean.npy"), mean)
        print(f"mean of {len(names)} images -> {os.path.join(a.out_dir, 'mean.npy')} "
              f"(per channel: {' '.join(f'{v:.4f}' for v in channel_mean(mean))})")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
