"""Tensor re-arrangements built from primitive layers
(python/lbann/modules/transformations.py:9-174)."""
from ..frontend import core as L


def Permute(x, dims, axes=None, name="", return_dims=False, avoid_gpu_permute=False):
    """Permute the sample dimensions ``dims`` of ``x`` by ``axes`` (default: reverse)."""
    axes = list(axes) if axes is not None else list(reversed(range(len(dims))))
    y = L.TensorPermute(x, axes=axes, name=name or None)
    new_dims = [dims[a] for a in axes]
    return (y, new_dims) if return_dims else y


def Cumsum(x, dims, axis=0):
    """Inclusive cumulative sum along ``axis`` of a 2-D tensor, as a product with a
    triangular matrix of ones (runs on the tensor-core GEMM)."""
    import numpy as np
    if len(dims) != 2:
        raise ValueError("Cumsum expects a 2-D tensor")
    n = dims[axis]
    tri = np.tril(np.ones((n, n), dtype=np.float32))
    w = L.Weights(initializer=L.ValueInitializer(values=tri.reshape(-1).tolist()), optimizer=L.NoOptimizer())
    t = L.WeightsLayer(weights=w, dims=[n, n])
    return L.MatMul(t, x) if axis == 0 else L.MatMul(x, t, transpose_b=True)


def _periodic(x, extent, axis, padding):
    pts = [0, padding, extent - padding, extent]
    s = L.Slice(x, axis=axis, slice_points=pts)
    head, mid, tail = L.Identity(s), L.Identity(s), L.Identity(s)
    inner = L.Concatenation([head, mid, tail], axis=axis)
    return L.Concatenation([tail, inner, head], axis=axis)


def PeriodicPadding2D(x, height, width, padding=1):
    """Wrap-around padding of a ``[C, H, W]`` tensor along H and W."""
    return _periodic(_periodic(x, height, 1, padding), width, 2, padding)


def PeriodicPadding3D(x, depth, height, width, padding=1):
    """Wrap-around padding of a ``[C, D, H, W]`` tensor along D, H and W."""
    y = _periodic(x, depth, 1, padding)
    return _periodic(_periodic(y, height, 2, padding), width, 3, padding)
