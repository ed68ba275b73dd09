"""Per-sample preprocessing pipeline (src/transforms/**, src/proto/transforms.proto).

Image transforms operate on HWC uint8/float arrays (OpenCV conventions) until
``to_lbann_layout`` / ``normalize_to_lbann_layout`` converts to CHW float32 in [0, 1];
the generic transforms (normalize, sample_normalize, scale) act on CHW float arrays.
"""
from __future__ import annotations

import math
from typing import Callable, List

import numpy as np


def _cv2():
    import cv2
    return cv2


def _floats(s):
    return [float(v) for v in (s.replace(",", " ").split() if isinstance(s, str) else s)]


class Pipeline:
    def __init__(self, steps: List[Callable], seed: int = 0):
        self.steps = steps
        self.rng = np.random.RandomState(seed or 1)

    def __call__(self, x):
        for s in self.steps:
            x = s(x, self.rng)
        return x


def _normalize(p):
    means, stds = np.asarray(_floats(p.means), np.float32), np.asarray(_floats(p.stddevs), np.float32)

    def f(x, rng):
        x = x.astype(np.float32, copy=False)
        shape = (-1,) + (1,) * (x.ndim - 1)
        return (x - means.reshape(shape)) / stds.reshape(shape)
    return f


def _sample_normalize(p):
    def f(x, rng):
        x = x.astype(np.float32, copy=False)
        sd = x.std()
        return (x - x.mean()) / (sd if sd > 0 else 1.0)
    return f


def _scale(p):
    s = float(p.scale)
    return lambda x, rng: x.astype(np.float32, copy=False) * s


def _to_layout(p):
    def f(x, rng):
        if x.ndim == 2:
            x = x[:, :, None]
        return np.ascontiguousarray(x.transpose(2, 0, 1)).astype(np.float32) / 255.0
    return f


def _normalize_to_layout(p):
    means, stds = np.asarray(_floats(p.means), np.float32), np.asarray(_floats(p.stddevs), np.float32)

    def f(x, rng):
        if x.ndim == 2:
            x = x[:, :, None]
        y = x.transpose(2, 0, 1).astype(np.float32) / 255.0
        return (y - means.reshape(-1, 1, 1)) / stds.reshape(-1, 1, 1)
    return f


def _resize(p):
    h, w = int(p.height), int(p.width)
    return lambda x, rng: _cv2().resize(x, (w, h), interpolation=_cv2().INTER_LINEAR)


def _center_crop_arr(x, h, w):
    H, W = x.shape[:2]
    t, l = max((H - h) // 2, 0), max((W - w) // 2, 0)
    return x[t:t + h, l:l + w]


def _center_crop(p):
    h, w = int(p.height), int(p.width)
    return lambda x, rng: _center_crop_arr(x, h, w)


def _resized_center_crop(p):
    h, w, ch, cw = int(p.height), int(p.width), int(p.crop_height), int(p.crop_width)
    return lambda x, rng: _center_crop_arr(_cv2().resize(x, (w, h)), ch, cw)


def _random_crop(p):
    h, w = int(p.height), int(p.width)

    def f(x, rng):
        H, W = x.shape[:2]
        t = rng.randint(0, max(H - h, 0) + 1)
        l = rng.randint(0, max(W - w, 0) + 1)
        return x[t:t + h, l:l + w]
    return f


def _random_resized_crop(p):
    h, w = int(p.height), int(p.width)
    smin, smax = float(p.scale_min) or 0.08, float(p.scale_max) or 1.0
    amin, amax = float(p.ar_min) or 0.75, float(p.ar_max) or 4.0 / 3.0

    def f(x, rng):
        H, W = x.shape[:2]
        for _ in range(10):
            area = H * W * rng.uniform(smin, smax)
            ar = math.exp(rng.uniform(math.log(amin), math.log(amax)))
            cw, ch = int(round(math.sqrt(area * ar))), int(round(math.sqrt(area / ar)))
            if 0 < cw <= W and 0 < ch <= H:
                t, l = rng.randint(0, H - ch + 1), rng.randint(0, W - cw + 1)
                return _cv2().resize(x[t:t + ch, l:l + cw], (w, h))
        return _cv2().resize(_center_crop_arr(x, min(H, W), min(H, W)), (w, h))
    return f


def _random_resized_crop_fixed(p):
    h, w, ch, cw = int(p.height), int(p.width), int(p.crop_height), int(p.crop_width)
    inner = _random_crop(type("P", (), {"height": ch, "width": cw}))
    return lambda x, rng: inner(_cv2().resize(x, (w, h)), rng)


def _hflip(p):
    prob = float(p.p) or 0.5
    return lambda x, rng: x[:, ::-1] if rng.rand() < prob else x


def _vflip(p):
    prob = float(p.p) or 0.5
    return lambda x, rng: x[::-1] if rng.rand() < prob else x


def _grayscale(p):
    return lambda x, rng: _cv2().cvtColor(x, _cv2().COLOR_BGR2GRAY)[:, :, None] if x.ndim == 3 and x.shape[2] == 3 else x


def _colorize(p):
    return lambda x, rng: _cv2().cvtColor(x, _cv2().COLOR_GRAY2BGR) if x.ndim == 2 or x.shape[2] == 1 else x


def _brightness(factor, x):
    return np.clip(x.astype(np.float32) * factor, 0, 255).astype(np.uint8)


def _contrast(factor, x):
    mean = x.astype(np.float32).mean()
    return np.clip((x.astype(np.float32) - mean) * factor + mean, 0, 255).astype(np.uint8)


def _saturation(factor, x):
    if x.ndim != 3 or x.shape[2] != 3:
        return x
    gray = _cv2().cvtColor(x, _cv2().COLOR_BGR2GRAY)[:, :, None].astype(np.float32)
    return np.clip((x.astype(np.float32) - gray) * factor + gray, 0, 255).astype(np.uint8)


def _color_jitter(p):
    def f(x, rng):
        ops = [
            lambda y: _brightness(rng.uniform(p.min_brightness_factor or 1, p.max_brightness_factor or 1), y),
            lambda y: _contrast(rng.uniform(p.min_contrast_factor or 1, p.max_contrast_factor or 1), y),
            lambda y: _saturation(rng.uniform(p.min_saturation_factor or 1, p.max_saturation_factor or 1), y)]
        for i in rng.permutation(3):
            x = ops[i](x)
        return x
    return f


def _cutout(p):
    holes, length = int(p.num_holes) or 1, int(p.length) or 1

    def f(x, rng):
        x = x.copy()
        H, W = x.shape[:2]
        for _ in range(holes):
            cy, cx = rng.randint(H), rng.randint(W)
            x[max(cy - length // 2, 0):cy + length // 2, max(cx - length // 2, 0):cx + length // 2] = 0
        return x
    return f


def _pad(p):
    n = int(p.pad)
    return lambda x, rng: np.pad(x, ((n, n), (n, n)) + ((0, 0),) * (x.ndim - 2))


def _random_affine(p):
    def f(x, rng):
        cv2 = _cv2()
        H, W = x.shape[:2]
        ang = rng.uniform(p.rotate_min, p.rotate_max)
        sc = rng.uniform(p.scale_min or 1.0, p.scale_max or 1.0)
        sh = math.radians(rng.uniform(p.shear_min, p.shear_max))
        tx = rng.uniform(-p.translate_w, p.translate_w) * W
        ty = rng.uniform(-p.translate_h, p.translate_h) * H
        m = cv2.getRotationMatrix2D((W / 2, H / 2), ang, sc)
        m[0, 1] += math.tan(sh)
        m[0, 2] += tx
        m[1, 2] += ty
        return cv2.warpAffine(x, m, (W, H))
    return f


_BUILDERS = {
    "normalize": _normalize, "sample_normalize": _sample_normalize, "scale": _scale,
    "to_lbann_layout": _to_layout, "normalize_to_lbann_layout": _normalize_to_layout,
    "resize": _resize, "center_crop": _center_crop, "resized_center_crop": _resized_center_crop,
    "random_crop": _random_crop, "random_resized_crop": _random_resized_crop,
    "random_resized_crop_with_fixed_aspect_ratio": _random_resized_crop_fixed,
    "horizontal_flip": _hflip, "vertical_flip": _vflip, "grayscale": _grayscale,
    "colorize": _colorize,
    "adjust_brightness": lambda p: (lambda x, rng: _brightness(float(p.factor), x)),
    "adjust_contrast": lambda p: (lambda x, rng: _contrast(float(p.factor), x)),
    "adjust_saturation": lambda p: (lambda x, rng: _saturation(float(p.factor), x)),
    "color_jitter": _color_jitter, "cutout": _cutout, "pad": _pad, "random_affine": _random_affine,
}


def build_pipeline(transform_msgs, seed: int = 0) -> Pipeline:
    steps = []
    for t in transform_msgs:
        which = t.WhichOneof("transform_type") if hasattr(t, "WhichOneof") else None
        if which is None:
            continue
        steps.append(_BUILDERS[which](getattr(t, which)))
    return Pipeline(steps, seed)
