"""Runtime weights: values in the model's parameter arena, initializers, per-weights
optimizer hyper-parameters.

Semantics follow the reference's ``weights`` / ``data_type_weights`` / ``optimizer``
classes (src/weights/data_type_weights.cpp:233-300, src/weights/initializer.cpp,
src/weights/variance_scaling_initializers.cpp, src/optimizers/*.cpp): every weights object
owns an initializer and (unless frozen or ``NoOptimizer``) a private copy of an optimizer
whose learning rate callbacks may change.  Storage differs by design: all weights of a
model are slices of one flat arena (see ``ops/optim.py``).
"""
from __future__ import annotations

import hashlib
import math
from typing import Optional

import numpy as np
import torch

from ..ops.nn import WeightHandle
from ..ops.optim import ParameterArena, Slot

OPT_DEFAULTS = {
    "sgd": {"learn_rate": 0.0, "momentum": 0.0, "nesterov": False},
    "adam": {"learn_rate": 0.0, "beta1": 0.9, "beta2": 0.99, "eps": 1e-8,
             "adamw_weight_decay": 0.0},
    "adagrad": {"learn_rate": 0.0, "eps": 1e-8},
    "rmsprop": {"learn_rate": 0.0, "decay_rate": 0.9, "eps": 1e-8},
    "hypergradient_adam": {"init_learning_rate": 0.0, "hyper_learning_rate": 1e-7, "beta1": 0.9,
                           "beta2": 0.99, "eps": 1e-8},
}


def optimizer_from_proto(opt_pb):
    """-> (kind, hyper-parameter dict) or (None, {}) when the message is empty."""
    which = opt_pb.WhichOneof("optimizer_type") if opt_pb is not None else None
    if which is None:
        return None, {}
    if which == "no_optimizer":
        return "none", {}
    msg = getattr(opt_pb, which)
    hp = dict(OPT_DEFAULTS.get(which, {}))
    for f in msg.DESCRIPTOR.fields:
        v = getattr(msg, f.name)
        # proto3 scalars: zero means "unset" for the fields that have non-zero defaults
        if f.name in ("beta1", "beta2", "eps", "decay_rate", "hyper_learning_rate") and v == 0:
            continue
        hp[f.name] = v
    if which == "hypergradient_adam":
        hp["learn_rate"] = hp.get("init_learning_rate", 0.0)
    return which, hp


class ExecWeights:
    """A named parameter tensor."""

    def __init__(self, name: str, proto=None):
        self.name = name
        self.proto = proto
        self.shape = None
        self.initializer = None           # callable(shape, generator) -> fp32 CPU tensor
        self.init_proto = proto.initializer if proto is not None and proto.HasField("initializer") else None
        self.opt_kind, self.opt_hp = (optimizer_from_proto(proto.optimizer)
                                      if proto is not None and proto.HasField("optimizer") else (None, {}))
        self.frozen = False
        self.sharded = bool(proto.sharded) if proto is not None else False
        self.sharding_strategy = int(proto.sharding_strategy) if proto is not None else 0
        self.fan_in = self.fan_out = None
        self.slot: Optional[Slot] = None
        self.handle: Optional[WeightHandle] = None
        self.arena: Optional[ParameterArena] = None
        self.users = []
        self.default_init = None          # set by the owning layer when no initializer is given
        self.hyper_state = None           # hypergradient Adam extras

    # ---- set-up
    def set_shape(self, shape, fan_in=None, fan_out=None):
        shape = tuple(int(s) for s in shape)
        if self.shape is not None and self.shape != shape:
            if math.prod(self.shape) != math.prod(shape):
                raise ValueError(f"weights '{self.name}' used with shapes {self.shape} and {shape}")
            return
        self.shape = shape
        if fan_in is not None:
            self.fan_in, self.fan_out = fan_in, fan_out

    def bind(self, arena: ParameterArena):
        self.arena = arena
        self.slot = arena.reserve(self.name, self.shape)

    def materialise(self, default_opt, seed: int):
        arena = self.arena
        master = arena.view(arena.master, self.slot)
        kind, hp = (self.opt_kind, self.opt_hp) if self.opt_kind is not None else default_opt
        if self.frozen:
            kind = "none"
        trainable = kind not in (None, "none")
        grad = arena.view(arena.grad, self.slot) if trainable else None
        compute = arena.view(arena.compute, self.slot) if arena.compute is not None else None
        values = self._initial_values(seed)
        with torch.no_grad():
            master.copy_(values.reshape(master.shape))
        if trainable:
            master.requires_grad_(True)
            # autograd accumulates into the arena slice in place
            master.grad = grad if grad.dtype == master.dtype else None
        self.handle = WeightHandle(master, grad, compute)
        self.slot.kind = kind or "none"
        self.slot.hp = dict(hp)
        self.opt_kind, self.opt_hp = kind or "none", self.slot.hp

    # ---- values
    def _generator(self, seed: int) -> torch.Generator:
        h = int(hashlib.sha1(self.name.encode()).hexdigest()[:8], 16)
        g = torch.Generator(device="cpu")
        g.manual_seed((int(seed) * 1000003 + h) % (2 ** 63 - 1))
        return g

    def _initial_values(self, seed: int) -> torch.Tensor:
        gen = self._generator(seed)
        n = int(math.prod(self.shape)) if self.shape else 1
        ip = self.init_proto
        which = ip.WhichOneof("initializer_type") if ip is not None else None
        if which is None:
            if self.default_init is not None:
                return self.default_init(self.shape, gen, self.fan_in, self.fan_out)
            return torch.zeros(n)
        msg = getattr(ip, which)
        if which == "constant_initializer":
            return torch.full((n,), float(msg.value))
        if which == "value_initializer":
            vals = list(msg.values) or list(msg.values_d)
            if len(vals) == 1:
                vals = vals * n
            if len(vals) != n:
                raise ValueError(f"weights '{self.name}': value initializer has {len(vals)} values "
                                 f"for {n} entries")
            return torch.tensor(vals, dtype=torch.float32)
        if which == "numpy_initializer":
            arr = np.load(msg.file)
            return torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).reshape(-1)
        if which == "uniform_initializer":
            lo, hi = float(msg.min), float(msg.max)
            if lo == 0.0 and hi == 0.0:
                hi = 1.0
            return torch.rand(n, generator=gen) * (hi - lo) + lo
        if which == "normal_initializer":
            sd = float(msg.standard_deviation) or 1.0
            return torch.randn(n, generator=gen) * sd + float(msg.mean)
        fan_in = self.fan_in or (self.shape[-1] if self.shape else 1)
        fan_out = self.fan_out or (self.shape[0] if self.shape else 1)
        return variance_scaling(which, n, fan_in, fan_out, gen)

    # ---- accessors
    @property
    def values(self) -> torch.Tensor:
        return self.handle.master

    @property
    def gradient(self) -> Optional[torch.Tensor]:
        return self.handle.grad

    def set_values(self, t: torch.Tensor):
        with torch.no_grad():
            self.handle.master.copy_(t.reshape(self.handle.master.shape).to(self.handle.master.dtype))
            if self.handle.compute16 is not None:
                self.handle.compute16.copy_(self.handle.master)
        self.handle.bump()

    def has_optimizer(self) -> bool:
        return self.slot is not None and self.slot.kind != "none"

    @property
    def learning_rate(self) -> float:
        return float(self.slot.hp.get("learn_rate", 0.0))

    @learning_rate.setter
    def learning_rate(self, v: float):
        self.slot.hp["learn_rate"] = float(v)

    def optimizer_state(self):
        """Dictionary of state tensors (views) for checkpointing / LTFB exchange."""
        out = {}
        if not self.has_optimizer():
            return out
        a = self.arena
        if self.slot.kind == "sgd":
            out["velocity"] = a.state_view(0, self.slot)
        elif self.slot.kind in ("adam", "hypergradient_adam"):
            a.ensure_state1()
            out["moment1"] = a.state_view(0, self.slot)
            out["moment2"] = a.state_view(1, self.slot)
            if self.slot.kind == "hypergradient_adam":
                if "old_gradient" not in self.slot.extra:
                    self.slot.extra["old_gradient"] = torch.zeros_like(a.view(a.master, self.slot))
                out["old_gradient"] = self.slot.extra["old_gradient"]
        else:
            out["cache"] = a.state_view(0, self.slot)
        return out


def variance_scaling(which: str, n: int, fan_in: float, fan_out: float, gen) -> torch.Tensor:
    """Glorot / He / LeCun initializers (normal or uniform)."""
    if which.startswith("glorot"):
        var = 2.0 / (fan_in + fan_out)
    elif which.startswith("he"):
        var = 2.0 / fan_in
    elif which.startswith("lecun"):
        var = 1.0 / fan_in
    else:
        raise ValueError(f"unknown initializer {which}")
    if "uniform" in which:
        lim = math.sqrt(3.0 * var)
        return (torch.rand(n, generator=gen) * 2 - 1) * lim
    return torch.randn(n, generator=gen) * math.sqrt(var)


def he_normal_default(shape, gen, fan_in, fan_out):
    n = int(math.prod(shape))
    return variance_scaling("he_normal_initializer", n, fan_in or shape[-1], fan_out or shape[0], gen)


def constant_default(value: float):
    def fn(shape, gen, fan_in, fan_out):
        return torch.full((int(math.prod(shape)) if shape else 1,), float(value))
    return fn
