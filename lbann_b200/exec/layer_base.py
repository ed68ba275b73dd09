"""Base class and registry of executable layers.

An executable layer is built from one ``lbann_data.Layer`` message.  ``setup`` derives the
output dimensions from the parents' (the mini-batch dimension is implicit, as in the
reference: src/proto/layers.proto:52-63) and creates default weights; ``forward`` maps a
list of input tensors ``[mini_batch, *dims]`` to a list of output tensors.  Backward
propagation is PyTorch autograd over those forward functions: the hot layers are custom
autograd functions around this library's kernels, the long tail is composed of PyTorch
operations.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..proto import lbann_pb2 as pb

LAYER_REGISTRY: Dict[str, type] = {}

_DTYPES = {
    pb.DataType.FLOAT: torch.float32,
    pb.DataType.DOUBLE: torch.float64,
    pb.DataType.FP16: torch.float16,
    pb.DataType.BF16: torch.bfloat16,
}



def rows2d(x):
    """[N, ...] -> [N, features]; also for a rank that holds no sample of the mini-batch
    (PyTorch cannot infer a -1 extent of an empty tensor)."""
    n = x.shape[0]
    if x.numel():
        return x.reshape(n, -1)
    f = 1
    for d in x.shape[1:]:
        f *= int(d)
    return x.reshape(n, f)


def register(*names):
    def deco(cls):
        for n in names:
            LAYER_REGISTRY[n] = cls
        cls.type_names = names
        return cls
    return deco


def prod(dims: Sequence[int]) -> int:
    return int(math.prod(dims)) if len(dims) else 1


def broadcast_list(values, n: int, default: int) -> Tuple[int, ...]:
    """Repeated field -> n-tuple (empty -> default, length 1 -> broadcast)."""
    v = [int(x) for x in values]
    if not v:
        return (default,) * n
    if len(v) == 1:
        return tuple(v) * n
    if len(v) != n:
        raise ValueError(f"expected {n} values, got {v}")
    return tuple(v)


class ExecLayer:
    """Executable counterpart of one layer message."""

    num_outputs = 1          # -1: one output per child
    min_parents = 1
    max_parents = 1          # -1: any number
    supports_distconv = False

    def __init__(self, proto, model):
        self.proto = proto
        self.model = model
        self.name = proto.name
        self.type = proto.WhichOneof("layer_type")
        self.params = getattr(proto, self.type) if self.type else None
        self.parent_names = list(proto.parents)
        self.child_names = list(proto.children)
        self.weight_names = list(proto.weights)
        self.hint_layer = proto.hint_layer or None
        self.data_layout = proto.data_layout or "data_parallel"
        self.frozen = bool(proto.freeze)
        if proto.HasField("grid_tag"):
            self.grid_tag = int(proto.grid_tag.value)
        elif proto.HasField("parallel_strategy") and proto.parallel_strategy.HasField("grid_tag"):
            self.grid_tag = int(proto.parallel_strategy.grid_tag.value)
        else:
            self.grid_tag = -1     # inherit from the parents (src/models/model.cpp:1041-1090)
        self.parallel_strategy = proto.parallel_strategy if proto.HasField("parallel_strategy") else None
        self.dtype = _DTYPES.get(proto.datatype, None)   # None -> model default
        self.parents: List["ExecLayer"] = []
        self.children: List["ExecLayer"] = []
        self.weights = []
        self.in_dims: List[Tuple[int, ...]] = []
        self.out_dims: List[Tuple[int, ...]] = []
        self.fp_time = 0.0
        self.bp_time = 0.0

    # ---- set-up
    def setup(self, in_dims: List[Tuple[int, ...]]) -> List[Tuple[int, ...]]:
        return [tuple(in_dims[0])] if in_dims else [()]

    def get_weights(self, index: int, suffix: str, shape, default_init=None, fan_in=None,
                    fan_out=None, optimizer: bool = True):
        """The index-th weights of this layer, created with the reference's default name
        (``<layer>_<suffix>``) when the user supplied none."""
        from .weights import ExecWeights
        if index < len(self.weight_names):
            w = self.model.weights_by_name[self.weight_names[index]]
        else:
            name = f"{self.name}_{suffix}"
            w = self.model.weights_by_name.get(name)
            if w is None:
                w = ExecWeights(name)
                self.model.add_weights(w)
            while len(self.weight_names) < index:
                self.weight_names.append("")
            self.weight_names.append(name)
        w.set_shape(shape, fan_in, fan_out)
        if w.default_init is None:
            w.default_init = default_init
        if not optimizer and w.opt_kind is None:
            w.opt_kind, w.opt_hp = "none", {}
        if self.frozen:
            w.frozen = True
        w.users.append(self)
        while len(self.weights) <= index:
            self.weights.append(None)
        self.weights[index] = w
        return w

    # ---- execution
    def forward(self, xs: List[torch.Tensor], training: bool) -> List[torch.Tensor]:
        raise NotImplementedError(self.type)

    def cast_in(self, x: torch.Tensor) -> torch.Tensor:
        dt = self.dtype or self.model.default_dtype
        if x.is_floating_point() and x.dtype != dt:
            return x.to(dt)
        return x

    def describe(self) -> str:
        s = f"{self.name} ({self.type}): in {self.in_dims} out {self.out_dims}"
        if self.parallel_strategy is not None:
            ps = self.parallel_strategy
            s += (f" strategy[n{ps.sample_groups} d{ps.depth_groups} h{ps.height_groups} "
                  f"w{ps.width_groups} c{ps.channel_groups} f{ps.filter_groups}]")
        return s
