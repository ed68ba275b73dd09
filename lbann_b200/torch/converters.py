"""Converters from ``torch.nn`` modules and tensor functions to front-end layers, and the
registries that ``register_module`` / ``register_function`` fill
(python/lbann/torch/converters.py, replacements/)."""
from __future__ import annotations

import operator
from typing import Callable, Dict, List

import numpy as np
import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

from ..frontend import core as L
from .helpers import _Ctx, _weights  # noqa: F401

_MODULES: Dict[type, Callable] = {}
_FUNCTIONS: Dict[object, Callable] = {}


def register_module(*classes):
    def deco(fn):
        for c in classes:
            _MODULES[c] = fn
        return fn
    return deco


def register_function(*fns):
    def deco(fn):
        for f in fns:
            _FUNCTIONS[f] = fn
        return fn
    return deco


@register_module(nn.Linear)
def _linear(m, name, ctx, x):
    ws = None
    if ctx.with_weights:
        ws = [_weights(m.weight, name + "_matrix")]      # [out, in], row-major like the layer's
        if m.bias is not None:
            ws.append(_weights(m.bias, name + "_bias"))
    rank = len(ctx.shapes[x]) if x in ctx.shapes else 1
    if rank > 1:
        return L.ChannelwiseFullyConnected(x, weights=ws, output_channel_dims=[m.out_features],
                                           bias=m.bias is not None, name=name)
    return L.FullyConnected(x, weights=ws, num_neurons=m.out_features, has_bias=m.bias is not None,
                            name=name)


@register_module(nn.Conv1d, nn.Conv2d, nn.Conv3d)
def _conv(m, name, ctx, x):
    ws = None
    if ctx.with_weights:
        ws = [_weights(m.weight, name + "_kernel")] + ([_weights(m.bias, name + "_bias")] if m.bias is not None else [])
    return L.Convolution(x, weights=ws, num_dims=len(m.kernel_size), out_channels=m.out_channels,
                         kernel_size=list(m.kernel_size), stride=list(m.stride), padding=list(m.padding),
                         dilation=list(m.dilation), groups=m.groups, has_bias=m.bias is not None, name=name)


@register_module(nn.ReLU)
def _relu(m, name, ctx, x):
    return L.Relu(x, name=name)


@register_module(nn.GELU)
def _gelu(m, name, ctx, x):
    return L.Gelu(x, name=name)


@register_module(nn.Tanh)
def _tanh(m, name, ctx, x):
    return L.Tanh(x, name=name)


@register_module(nn.Sigmoid)
def _sigmoid(m, name, ctx, x):
    return L.Sigmoid(x, name=name)


@register_module(nn.LeakyReLU)
def _leaky(m, name, ctx, x):
    return L.LeakyRelu(x, negative_slope=m.negative_slope, name=name)


@register_module(nn.Dropout)
def _dropout(m, name, ctx, x):
    return L.Dropout(x, keep_prob=1 - m.p, name=name)


@register_module(nn.Identity)
def _identity(m, name, ctx, x):
    return L.Identity(x, name=name)


@register_module(nn.Flatten)
def _flatten(m, name, ctx, x):
    return L.Reshape(x, dims=[-1], name=name)


@register_module(nn.MaxPool2d, nn.AvgPool2d, nn.MaxPool3d, nn.AvgPool3d)
def _pool(m, name, ctx, x):
    nd = 3 if isinstance(m, (nn.MaxPool3d, nn.AvgPool3d)) else 2
    v = lambda a: list(a) if isinstance(a, (tuple, list)) else [a] * nd   # noqa: E731
    mode = "max" if isinstance(m, (nn.MaxPool2d, nn.MaxPool3d)) else "average"
    return L.Pooling(x, num_dims=nd, has_vectors=True, pool_dims=v(m.kernel_size),
                     pool_strides=v(m.stride or m.kernel_size), pool_pads=v(m.padding), pool_mode=mode,
                     name=name)


@register_module(nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d)
def _bn(m, name, ctx, x):
    ws = None
    if ctx.with_weights:
        ws = [_weights(m.weight, name + "_scale"), _weights(m.bias, name + "_bias"),
              _weights(m.running_mean, name + "_running_mean", False),
              _weights(m.running_var, name + "_running_variance", False)]
    return L.BatchNormalization(x, weights=ws, decay=1 - (m.momentum or 0.1), epsilon=m.eps, name=name)


@register_module(nn.LayerNorm)
def _ln(m, name, ctx, x):
    ws = None
    if ctx.with_weights and m.elementwise_affine:
        ws = [_weights(m.weight, name + "_weight"), _weights(m.bias, name + "_bias")]
    return L.LayerNorm(x, epsilon=m.eps, scale=m.elementwise_affine, bias=m.elementwise_affine,
                       start_dim=-len(m.normalized_shape), weights=ws, name=name)


@register_module(nn.Softmax)
def _softmax(m, name, ctx, x):
    return L.Softmax(x, name=name)


@register_function(torch.relu, F.relu)
def _f_relu(name, ctx, x, *a, **k):
    return L.Relu(x, name=name)


@register_function(torch.tanh, F.tanh)
def _f_tanh(name, ctx, x):
    return L.Tanh(x, name=name)


@register_function(torch.sigmoid, F.sigmoid)
def _f_sigmoid(name, ctx, x):
    return L.Sigmoid(x, name=name)


@register_function(F.gelu)
def _f_gelu(name, ctx, x, **k):
    return L.Gelu(x, name=name)


@register_function(operator.add, torch.add)
def _f_add(name, ctx, a, b):
    if isinstance(b, (int, float)):
        return L.AddConstant(a, constant=float(b), name=name)
    return L.Add(a, b, name=name)


@register_function(operator.sub, torch.sub)
def _f_sub(name, ctx, a, b):
    if isinstance(b, (int, float)):
        return L.AddConstant(a, constant=-float(b), name=name)
    return L.Subtract(a, b, name=name)


@register_function(operator.mul, torch.mul)
def _f_mul(name, ctx, a, b):
    if isinstance(b, (int, float)):
        return L.Scale(a, constant=float(b), name=name)
    if isinstance(a, (int, float)):
        return L.Scale(b, constant=float(a), name=name)
    return L.Multiply(a, b, name=name)


@register_function(torch.flatten)
def _f_flatten(name, ctx, x, *a, **k):
    return L.Reshape(x, dims=[-1], name=name)


@register_module(nn.ConvTranspose1d, nn.ConvTranspose2d, nn.ConvTranspose3d)
def _deconv(m, name, ctx, x):
    ws = None
    if ctx.with_weights:
        ws = [_weights(m.weight, name + "_kernel")] + ([_weights(m.bias, name + "_bias")] if m.bias is not None else [])
    return L.Deconvolution(x, weights=ws, num_dims=len(m.kernel_size), out_channels=m.out_channels,
                           kernel_size=list(m.kernel_size), stride=list(m.stride), padding=list(m.padding),
                           output_padding=list(m.output_padding), dilation=list(m.dilation), groups=m.groups,
                           has_bias=m.bias is not None, name=name)


@register_module(nn.Embedding)
def _embedding(m, name, ctx, x):
    ws = [_weights(m.weight, name + "_table")] if ctx.with_weights else None
    return L.Embedding(x, weights=ws, num_embeddings=m.num_embeddings, embedding_dim=m.embedding_dim,
                       padding_idx=-1 if m.padding_idx is None else m.padding_idx, name=name)


@register_module(nn.AdaptiveAvgPool2d, nn.AdaptiveAvgPool3d)
def _global_pool(m, name, ctx, x):
    size = m.output_size if isinstance(m.output_size, (tuple, list)) else (m.output_size,)
    if any(v not in (1, None) for v in size):
        raise NotImplementedError("lbann.torch: adaptive pooling is lowered for output size 1 only")
    shape = ctx.shapes.get(x)
    y = L.ChannelwiseMean(x, name=name)
    return L.Reshape(y, dims=[shape[0]] + [1] * (len(shape) - 1), name=name + "_shape") if shape else y


@register_module(nn.ELU)
def _elu(m, name, ctx, x):
    return L.Elu(x, alpha=m.alpha, name=name)


@register_module(nn.SiLU)
def _silu(m, name, ctx, x):
    return L.Multiply(x, L.Sigmoid(x, name=name + "_gate"), name=name)


@register_module(nn.LogSoftmax)
def _logsoftmax(m, name, ctx, x):
    return L.LogSoftmax(x, name=name)


def _sample_dim(ctx, x, dim):
    """A tensor dimension (mini-batch first, negative allowed) as a sample dimension."""
    rank = len(ctx.shapes[x]) + 1
    d = dim % rank
    if d == 0:
        raise NotImplementedError("lbann.torch: operations along the mini-batch dimension are not lowered")
    return d - 1


@register_function(torch.cat, torch.concat)
def _f_cat(name, ctx, tensors, dim=0):
    tensors = list(tensors)
    return L.Concatenation(tensors, axis=_sample_dim(ctx, tensors[0], dim), name=name)


@register_function(torch.matmul, operator.matmul)
def _f_matmul(name, ctx, a, b):
    return L.MatMul(a, b, name=name)


@register_function(torch.reshape, torch.Tensor.reshape, torch.Tensor.view)
def _f_reshape(name, ctx, x, *shape):
    shape = list(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)) else list(shape)
    return L.Reshape(x, dims=[int(v) for v in shape[1:]], name=name)       # the first entry is the mini-batch


@register_function(torch.permute, torch.Tensor.permute)
def _f_permute(name, ctx, x, *dims):
    dims = list(dims[0]) if len(dims) == 1 and isinstance(dims[0], (tuple, list)) else list(dims)
    if dims[0] != 0:
        raise NotImplementedError("lbann.torch: the mini-batch dimension must stay first in a permutation")
    return L.TensorPermute(x, axes=[d - 1 for d in dims[1:]], name=name)


@register_function(torch.transpose, torch.Tensor.transpose)
def _f_transpose(name, ctx, x, d0, d1):
    rank = len(ctx.shapes[x])
    axes = list(range(rank))
    a, b = _sample_dim(ctx, x, d0), _sample_dim(ctx, x, d1)
    axes[a], axes[b] = axes[b], axes[a]
    return L.TensorPermute(x, axes=axes, name=name)


@register_function(torch.mean, torch.Tensor.mean)
def _f_mean(name, ctx, x, dim=None, keepdim=False):
    shape = ctx.shapes[x]
    dims = list(range(1, len(shape) + 1)) if dim is None else ([dim] if isinstance(dim, int) else list(dim))
    dims = sorted(_sample_dim(ctx, x, d) for d in dims)
    if dims == list(range(len(shape))):
        return L.Reduction(x, mode="mean", name=name)
    if dims == list(range(1, len(shape))):
        y = L.ChannelwiseMean(x, name=name)
        return L.Reshape(y, dims=[shape[0]] + [1] * (len(shape) - 1), name=name + "_keep") if keepdim else y
    if len(dims) == 1:
        # one dimension: bring it to the front and multiply by a constant row of 1 / extent
        d = dims[0]
        axes = [d] + [a for a in range(len(shape)) if a != d]
        rest = [shape[a] for a in axes[1:]]
        n_rest = 1
        for v in rest:
            n_rest *= v
        y = x if d == 0 else L.TensorPermute(x, axes=axes, name=name + "_front")
        y = L.Reshape(y, dims=[shape[d], n_rest], name=name + "_2d")
        row = L.Constant(value=1.0 / shape[d], num_neurons=[1, shape[d]], name=name + "_row")
        y = L.MatMul(row, y, name=name + "_sum")
        out = list(shape)
        if keepdim:
            out[d] = 1
        else:
            del out[d]
        return L.Reshape(y, dims=out, name=name)
    raise NotImplementedError("lbann.torch: mean over one sample dimension, over all, or over all but the first")


@register_function(F.softmax, torch.softmax, torch.Tensor.softmax)
def _f_softmax(name, ctx, x, dim=-1, **k):
    shape = ctx.shapes[x]
    d = _sample_dim(ctx, x, dim)
    if len(shape) == 1:
        return L.Softmax(x, name=name)
    if d == len(shape) - 1:
        return L.ChannelwiseSoftmax(x, dim=-1, name=name) if len(shape) > 2 else L.ChannelwiseSoftmax(x, name=name)
    if d == 0:
        return L.Softmax(x, softmax_mode="channel", name=name)
    raise NotImplementedError("lbann.torch: softmax over the first or the last sample dimension only")


@register_function(operator.truediv, torch.div)
def _f_div(name, ctx, a, b):
    if isinstance(b, (int, float)):
        return L.Scale(a, constant=1.0 / float(b), name=name)
    return L.Divide(a, b, name=name)


@register_function(operator.neg, torch.neg)
def _f_neg(name, ctx, x):
    return L.Negative(x, name=name)


@register_function(torch.exp)
def _f_exp(name, ctx, x):
    return L.Exp(x, name=name)


@register_function(torch.sqrt)
def _f_sqrt(name, ctx, x):
    return L.Sqrt(x, name=name)


@register_function(F.silu)
def _f_silu(name, ctx, x, **k):
    return L.Multiply(x, L.Sigmoid(x, name=name + "_gate"), name=name)


@register_function(F.leaky_relu)
def _f_leaky(name, ctx, x, negative_slope=0.01, **k):
    return L.LeakyRelu(x, negative_slope=negative_slope, name=name)
