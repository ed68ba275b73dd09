"""Callback hook interface and the registry keyed by the ``Callback`` oneof field name.

Hook set and ``batch_interval`` semantics follow include/lbann/callbacks/callback.hpp:76-193.
"""
from __future__ import annotations

from typing import Dict

CALLBACK_REGISTRY: Dict[str, type] = {}


def register(*names):
    def deco(cls):
        for n in names:
            CALLBACK_REGISTRY[n] = cls
        return cls
    return deco


class ExecCallback:
    """Every hook is a no-op by default.  ``model.ctx`` is the current execution context
    (epoch, step, mode) and ``model.trainer`` the owning trainer."""

    batch_interval = 1

    def __init__(self, params=None):
        self.params = params
        bi = getattr(params, "batch_interval", 0) if params is not None else 0
        self.batch_interval = int(bi) if bi else 1

    # set-up
    def setup_trainer(self, trainer): pass
    def setup(self, model): pass
    def on_setup_begin(self, model): pass
    def on_setup_end(self, model): pass
    # training
    def on_train_begin(self, model): pass
    def on_train_end(self, model): pass
    def on_phase_end(self, model): pass
    def on_epoch_begin(self, model): pass
    def on_epoch_end(self, model): pass
    def on_batch_begin(self, model): pass
    def on_batch_end(self, model): pass
    # evaluation
    def on_validation_begin(self, model): pass
    def on_validation_end(self, model): pass
    def on_test_begin(self, model): pass
    def on_test_end(self, model): pass
    def on_batch_evaluate_begin(self, model, mode): pass
    def on_batch_evaluate_end(self, model, mode): pass
    # propagation
    def on_forward_prop_begin(self, model, mode): pass
    def on_forward_prop_end(self, model, mode): pass
    def on_layer_forward_begin(self, model, layer, mode): pass
    def on_layer_forward_end(self, model, layer, mode): pass
    def on_backward_prop_begin(self, model): pass
    def on_backward_prop_end(self, model): pass
    def on_optimize_begin(self, model): pass
    def on_optimize_end(self, model): pass


def build_callback(cb_pb):
    which = cb_pb.WhichOneof("callback_type")
    if which is None:
        raise ValueError("empty callback message")
    if which not in CALLBACK_REGISTRY:
        raise NotImplementedError(f"callback '{which}' is not available")
    return CALLBACK_REGISTRY[which](getattr(cb_pb, which))


def is_master(model) -> bool:
    return model.comm is None or model.comm.am_world_master()


def is_trainer_master(model) -> bool:
    return model.comm is None or model.comm.am_trainer_master()


def mode_string(model, mode=None) -> str:
    ctx = model.ctx
    mode = mode or ctx.mode
    if mode == "training":
        return f"training epoch {ctx.epoch}"
    return {"testing": "test"}.get(mode, mode)


def select_weights(model, names: str):
    names = names.split() if isinstance(names, str) else list(names)
    if not names:
        return [w for w in model.weights if w.has_optimizer()]
    return [model.weights_by_name[n] for n in names if n in model.weights_by_name]


def select_layers(model, names: str):
    names = names.split() if isinstance(names, str) else list(names)
    if not names:
        return list(model.layers)
    return [model.layers_by_name[n] for n in names if n in model.layers_by_name]
