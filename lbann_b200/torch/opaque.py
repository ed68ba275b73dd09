"""Tracing with opaque modules (python/lbann/torch/opaque.py): a module class that has a
registered converter is kept as ONE node of the traced graph instead of being traced into,
whether it comes from ``torch.nn`` or from user code (whose ``forward`` may not be traceable
at all: data-dependent control flow, calls into extensions)."""
from __future__ import annotations

import torch.fx as fx
import torch.nn as nn


class OpaqueTracer(fx.Tracer):
    def is_leaf_module(self, m: nn.Module, module_qualified_name: str) -> bool:
        from .converters import _MODULES
        return type(m) in _MODULES or super().is_leaf_module(m, module_qualified_name)


def trace(module: nn.Module) -> fx.GraphModule:
    tracer = OpaqueTracer()
    graph = tracer.trace(module)
    return fx.GraphModule(tracer.root, graph, module.__class__.__name__)


def register_opaque(*classes):
    """Decorator: ``fn(module, name, ctx, *inputs) -> layer`` lowers instances of ``classes``
    as a whole (the same registry as ``register_module``; the name says what it is for)."""
    from .converters import register_module
    return register_module(*classes)
