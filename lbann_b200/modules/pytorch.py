"""Layer patterns with PyTorch's calling conventions (python/lbann/modules/pytorch.py):
batched matrix products over leading dimensions, ``nn.Linear`` on tensors of any rank and
``nn.LayerNorm`` over the last dimension.  Shapes are sample shapes (no mini-batch entry)."""
from __future__ import annotations

from math import prod

from ..frontend import core as L


def PytorchMatmul(x, x_shape, y, y_shape, return_dims=False):
    """``torch.matmul`` of two tensors of equal rank: the leading dimensions are batched."""
    x_shape, y_shape = tuple(x_shape), tuple(y_shape)
    if len(x_shape) != len(y_shape):
        raise RuntimeError("broadcasting is not implemented: both tensors must have the same rank")
    if len(x_shape) > 3:
        if x_shape[:-2] != y_shape[:-2]:
            raise RuntimeError("the leading dimensions of both tensors must match")
        x = L.Reshape(x, dims=[prod(x_shape[:-2])] + list(x_shape[-2:]))
        y = L.Reshape(y, dims=[prod(y_shape[:-2])] + list(y_shape[-2:]))
    z = L.MatMul(x, y)
    z_shape = x_shape[:-1] + (y_shape[-1],)
    if len(x_shape) > 3:
        z = L.Reshape(z, dims=list(z_shape))
    return (z, z_shape) if return_dims else z


def PytorchLinear(x, input_shape, hidden_size, weights=(), name="", return_dims=False):
    """``nn.Linear`` applied to the last dimension of a tensor of any rank."""
    input_shape = tuple(input_shape)
    kw = {"name": name} if name else {}
    if weights:
        kw["weights"] = list(weights)
    if len(input_shape) == 1:
        y = L.FullyConnected(x, num_neurons=hidden_size, **kw)
        out = (hidden_size,)
    else:
        if len(input_shape) > 2:
            x = L.Reshape(x, dims=[prod(input_shape[:-1]), input_shape[-1]])
        y = L.ChannelwiseFullyConnected(x, output_channel_dims=[hidden_size], **kw)
        out = input_shape[:-1] + (hidden_size,)
        if len(input_shape) > 2:
            y = L.Reshape(y, dims=list(out))
    return (y, out) if return_dims else y


def PytorchLayerNorm(x, epsilon, input_shape, weights=(), name=""):
    """``nn.LayerNorm`` over the last dimension with a learned scale and bias."""
    input_shape = tuple(input_shape)
    kw = {"name": name} if name else {}
    if weights:
        kw["weights"] = list(weights)
    if len(input_shape) > 2:
        x = L.Reshape(x, dims=[prod(input_shape[:-1]), input_shape[-1]])
    y = L.LayerNorm(x, epsilon=epsilon, scale=True, bias=True, start_dim=-1, **kw)
    if len(input_shape) > 2:
        y = L.Reshape(y, dims=list(input_shape))
    return y
