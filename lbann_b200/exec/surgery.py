"""Model surgery: insert, remove, replace and swap layers of a model that is already set up.

The reference edits the layer list in place and re-runs the parts of setup that the edit
invalidates (``model::insert_layer / remove_layer / replace_layer / swap_layers``,
src/models/model.cpp:493-640; used by the LTFB mutation strategies and by callbacks that
rewrite the graph).  Here every tensor of a model (weights, gradients, optimizer state) sits in
one flat arena whose layout follows the layer list, so an edit is made on the model's
prototext and the model is built again from it; weights that keep their name and shape take
their values, optimizer state and hyper-parameters over.  Collective over the trainer when the
optimizer state is sharded (every rank makes the same edit).

    new_model = surgery.replace_layer(trainer, model, "act1", lbann_layer_pb)

The returned model replaces the old one in ``trainer.models``.
"""
from __future__ import annotations

from typing import Callable, Optional

from ..proto import lbann_pb2 as pb
from .ltfb import pack_model, unpack_model
from .model import LbannError


def _find(model_pb, name: str) -> int:
    for i, l in enumerate(model_pb.layer):
        if l.name == name:
            return i
    raise LbannError(f"model surgery: no layer named '{name}'")


def _set(field, names) -> None:
    del field[:]
    field.extend(names)


def _rename_in(field, old: str, new) -> None:
    """In a repeated name field: every ``old`` becomes ``new`` (a name, a list of names, or
    None to drop it)."""
    out = []
    for n in field:
        if n != old:
            out.append(n)
        elif isinstance(new, (list, tuple)):
            out.extend(new)
        elif new is not None:
            out.append(new)
    _set(field, out)


def _edit(trainer, model, edit: Callable[[pb.Model], None]):
    new_pb = pb.Model()
    new_pb.CopyFrom(model.proto)
    edit(new_pb)
    state = pack_model(model, with_optimizer=True)
    old_ctx = {k[1]: v for k, v in trainer.contexts.items() if k[0] == id(model)}
    if model in trainer.models:
        trainer.models.remove(model)
    for mode in old_ctx:
        del trainer.contexts[(id(model), mode)]
    new_model = trainer.build_model(new_pb)
    for mode, ctx in old_ctx.items():           # the run carries on where it was
        trainer.contexts[(id(new_model), mode)] = ctx
    if "training" in old_ctx:
        new_model.ctx = old_ctx["training"]
    keep = {}
    for w in new_model.weights:
        v = state.get(f"{w.name}/values")
        if v is not None and tuple(v.shape) == tuple(w.values.shape):
            for k, t in state.items():
                if k.startswith(w.name + "/"):
                    keep[k] = t
    unpack_model(new_model, keep, with_optimizer=True)
    return new_model


def insert_layer(trainer, model, layer_pb, after: str):
    """``layer_pb`` (name and type filled in; parents / children are set here) goes between
    layer ``after`` and all of its children."""
    def edit(m):
        i = _find(m, after)
        if any(l.name == layer_pb.name for l in m.layer):
            raise LbannError(f"model surgery: a layer named '{layer_pb.name}' exists already")
        new = pb.Layer()
        new.CopyFrom(layer_pb)
        _set(new.parents, [after])
        _set(new.children, list(m.layer[i].children))
        for l in m.layer:
            if l.name != after:
                _rename_in(l.parents, after, new.name)
        if len(m.layer[i].children):
            _set(m.layer[i].children, [new.name])
        layers = [pb.Layer() for _ in m.layer]
        for dst, src in zip(layers, m.layer):
            dst.CopyFrom(src)
        layers.insert(i + 1, new)
        del m.layer[:]
        m.layer.extend(layers)
    return _edit(trainer, model, edit)


def remove_layer(trainer, model, name: str):
    """Takes out a layer with one parent; its children read from that parent instead."""
    def edit(m):
        i = _find(m, name)
        parents = list(m.layer[i].parents)
        if len(parents) != 1:
            raise LbannError(f"model surgery: cannot remove '{name}' with {len(parents)} parents")
        for term in m.objective_function.layer_term:
            if term.layer == name:
                raise LbannError(f"model surgery: '{name}' is an objective term")
        parent, kids = parents[0], list(m.layer[i].children)
        for l in m.layer:
            if l.name == name:
                continue
            _rename_in(l.parents, name, parent)
            _rename_in(l.children, name, kids if l.name == parent else None)
        del m.layer[i]
    return _edit(trainer, model, edit)


def replace_layer(trainer, model, name: str, layer_pb):
    """The layer called ``name`` becomes ``layer_pb`` (which may carry another name); edges,
    objective terms and metrics that named the old layer follow."""
    def edit(m):
        i = _find(m, name)
        new = pb.Layer()
        new.CopyFrom(layer_pb)
        if not new.name:
            new.name = name
        if new.name != name and any(l.name == new.name for l in m.layer):
            raise LbannError(f"model surgery: a layer named '{new.name}' exists already")
        _set(new.parents, list(m.layer[i].parents))
        _set(new.children, list(m.layer[i].children))
        m.layer[i].CopyFrom(new)
        if new.name != name:
            for l in m.layer:
                _rename_in(l.parents, name, new.name)
                _rename_in(l.children, name, new.name)
            for term in m.objective_function.layer_term:
                if term.layer == name:
                    term.layer = new.name
            for metric in m.metric:
                if metric.HasField("layer_metric") and metric.layer_metric.layer == name:
                    metric.layer_metric.layer = new.name
    return _edit(trainer, model, edit)


def swap_layers(trainer, model, first: str, second: str):
    """Two layers exchange their places in the graph (each takes the other's edges)."""
    def edit(m):
        i, j = _find(m, first), _find(m, second)
        tmp = "\x00swap"

        def ren(field):
            _rename_in(field, first, tmp)
            _rename_in(field, second, first)
            _rename_in(field, tmp, second)
        for l in m.layer:
            ren(l.parents)
            ren(l.children)
        pi, ci = list(m.layer[i].parents), list(m.layer[i].children)
        _set(m.layer[i].parents, list(m.layer[j].parents))
        _set(m.layer[i].children, list(m.layer[j].children))
        _set(m.layer[j].parents, pi)
        _set(m.layer[j].children, ci)
    return _edit(trainer, model, edit)
