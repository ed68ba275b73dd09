"""fx-based lowering of PyTorch modules to front-end layers."""
from __future__ import annotations

import operator
from typing import Callable, Dict, List

import numpy as np
import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

from ..frontend import core as L

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


def _weights(t: torch.Tensor, name: str, trainable: bool = True):
    vals = t.detach().float().cpu().numpy()
    return L.Weights(initializer=L.ValueInitializer(values=vals.reshape(-1).tolist()), name=name,
                     optimizer=None if trainable else L.NoOptimizer())


class _Ctx:
    def __init__(self, with_weights):
        self.with_weights = with_weights
        self.shapes = {}


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


def compile(module: nn.Module, with_weights: bool = True, **example_inputs) -> List[L.Layer]:
    """Lower ``module`` to LBANN layers.  ``example_inputs`` maps the module's argument names
    to example tensors WITH the mini-batch dimension (used for shape propagation); every
    argument becomes an ``lbann.Input`` on the data field of the same name (the first one
    on ``samples``).  Returns the list of output layers."""
    gm = fx.symbolic_trace(module)
    ctx = _Ctx(with_weights)
    # shape propagation (sample shapes, without the batch dimension)
    from torch.fx.passes.shape_prop import ShapeProp
    names = [n.target for n in gm.graph.nodes if n.op == "placeholder"]
    if example_inputs:
        vals = list(example_inputs.values())
        ShapeProp(gm).propagate(*[example_inputs.get(n, vals[i] if i < len(vals) else None)
                                  for i, n in enumerate(names)])
    env: Dict[str, object] = {}
    mods = dict(gm.named_modules())
    outputs: List[L.Layer] = []
    first = True
    for node in gm.graph.nodes:
        lname = "torch_" + node.name
        if node.op == "placeholder":
            layer = L.Input(data_field="samples" if first else node.name, name=lname)
            first = False
        elif node.op == "call_module":
            m = mods[node.target]
            conv = _MODULES.get(type(m))
            if conv is None:
                raise NotImplementedError(f"lbann.torch: no converter for module {type(m).__name__} "
                                          f"(node '{node.name}')")
            args = [env[a.name] if isinstance(a, fx.Node) else a for a in node.args]
            layer = conv(m, lname, ctx, *args)
        elif node.op == "call_function" or node.op == "call_method":
            key = node.target if node.op == "call_function" else getattr(torch.Tensor, node.target, None)
            conv = _FUNCTIONS.get(key) or _FUNCTIONS.get(getattr(torch, str(node.target), None))
            if conv is None:
                raise NotImplementedError(f"lbann.torch: no converter for function {node.target} "
                                          f"(node '{node.name}')")
            args = [env[a.name] if isinstance(a, fx.Node) else a for a in node.args]
            kwargs = {k: (env[v.name] if isinstance(v, fx.Node) else v) for k, v in node.kwargs.items()}
            layer = conv(lname, ctx, *args, **kwargs)
        elif node.op == "output":
            outs = node.args[0]
            outs = outs if isinstance(outs, (tuple, list)) else [outs]
            outputs = [env[o.name] for o in outs]
            continue
        else:
            raise NotImplementedError(f"lbann.torch: unsupported fx node kind {node.op}")
        env[node.name] = layer
        meta = node.meta.get("tensor_meta")
        if meta is not None:
            ctx.shapes[layer] = tuple(meta.shape[1:])
    return outputs
