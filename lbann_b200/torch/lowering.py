"""Walk of a traced ``torch.fx`` graph that emits front-end layers node by node
(python/lbann/torch/lowering.py)."""
from __future__ import annotations

import operator
from typing import Callable, Dict, List

import numpy as np
import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

from ..frontend import core as L
from .converters import _FUNCTIONS, _MODULES
from .helpers import _Ctx, _weights
from .opaque import trace


def compile(module: nn.Module, with_weights: bool = True, **example_inputs) -> List[L.Layer]:
    """Lower ``module`` to LBANN layers.  ``example_inputs`` maps the module's argument names
    to example tensors WITH the mini-batch dimension (used for shape propagation); every
    argument becomes an ``lbann.Input`` on the data field of the same name (the first one
    on ``samples``).  Returns the list of output layers."""
    gm = trace(module)
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
            if node.op == "call_method" and key not in _FUNCTIONS and node.target in ("size", "contiguous"):
                if node.target == "contiguous":
                    env[node.name] = env[node.args[0].name]
                    ctx.shapes.setdefault(env[node.name], ctx.shapes.get(env[node.args[0].name]))
                    continue
                raise NotImplementedError("lbann.torch: shapes must be static (x.size() in forward)")
            conv = _FUNCTIONS.get(key) or _FUNCTIONS.get(getattr(torch, str(node.target), None))
            if conv is None:
                raise NotImplementedError(f"lbann.torch: no converter for function {node.target} "
                                          f"(node '{node.name}')")
            args = fx.node.map_arg(node.args, lambda n: env[n.name])          # also inside lists / tuples
            kwargs = fx.node.map_arg(node.kwargs, lambda n: env[n.name])
            layer = conv(lname, ctx, *args, **kwargs)
        elif node.op == "get_attr":
            t = gm
            for part in str(node.target).split("."):
                t = getattr(t, part)
            if not isinstance(t, torch.Tensor):
                raise NotImplementedError(f"lbann.torch: attribute '{node.target}' is not a tensor")
            trainable = isinstance(t, nn.Parameter) and t.requires_grad
            w = _weights(t, lname + "_values", trainable) if with_weights else \
                L.Weights(name=lname + "_values", optimizer=None if trainable else L.NoOptimizer())
            layer = L.WeightsLayer(weights=w, dims=list(t.shape), name=lname)
            env[node.name] = layer
            ctx.shapes[layer] = tuple(t.shape)           # a parameter has no mini-batch dimension
            continue
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
