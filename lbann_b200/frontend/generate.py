"""Descriptor-driven class generation for the Python front end.

Every member of a protobuf ``oneof`` (layer types, optimizers, callbacks, initializers,
operators ...) becomes a Python class whose keyword arguments are the message's fields,
with nested enums exposed as class attributes and an ``export_proto()`` method.  The
reference builds its front end the same way (python/lbann/core/util.py:62-233); this is
an independent implementation over the in-process schema.
"""
from __future__ import annotations

from google.protobuf import message as _pbmessage

_WRAPPERS = {"DoubleValue", "FloatValue", "Int64Value", "UInt64Value", "Int32Value",
             "UInt32Value", "BoolValue", "StringValue", "BytesValue"}


def make_iterable(obj):
    """Scalars (and strings) become 1-tuples; iterables are returned as they are."""
    if isinstance(obj, (str, bytes)):
        return (obj,)
    try:
        iter(obj)
        return obj
    except TypeError:
        return (obj,)


def str_list(values, sep: str = " ") -> str:
    """Space-separated string form used by many schema fields."""
    if isinstance(values, str):
        return values
    return sep.join(str(v) for v in make_iterable(values))


def set_message(msg, **kwargs):
    """Assign keyword values to a protobuf message, converting front-end objects."""
    fields = msg.DESCRIPTOR.fields_by_name
    for key, value in kwargs.items():
        if key not in fields:
            raise KeyError(f"message {msg.DESCRIPTOR.name} has no field '{key}'")
        if value is None:
            continue
        fd = fields[key]
        try:
            if fd.message_type is not None and fd.message_type.name in _WRAPPERS and \
                    fd.message_type.full_name.startswith("google.protobuf."):
                getattr(msg, key).value = value
            elif fd.is_repeated if hasattr(fd, "is_repeated") else fd.label == fd.LABEL_REPEATED:
                target = getattr(msg, key)
                items = list(make_iterable(value))
                if fd.message_type is not None:
                    for it in items:
                        target.add().CopyFrom(it.export_proto() if hasattr(it, "export_proto") else it)
                else:
                    target.extend(items)
            elif isinstance(value, _pbmessage.Message):
                getattr(msg, key).CopyFrom(value)
            elif hasattr(value, "export_proto"):
                getattr(msg, key).CopyFrom(value.export_proto())
            elif fd.message_type is not None and isinstance(value, dict):
                set_message(getattr(msg, key), **value)
                getattr(msg, key).SetInParent()
            else:
                if fd.type == fd.TYPE_STRING and not isinstance(value, str):
                    value = str_list(value)
                setattr(msg, key, value)
        except (TypeError, ValueError, AttributeError) as exc:
            raise TypeError(f"cannot set field '{key}' of {msg.DESCRIPTOR.name} from "
                            f"{type(value).__name__}: {exc}") from exc


def _enum_namespace(desc):
    return type(desc.name, (), {v.name: v.number for v in desc.values})


def class_from_message(desc, parent_field, base, base_kwargs, parent_message_cls=None):
    """Build a front-end class for message ``desc``.

    ``parent_field`` is the field of the base class's message that holds this message
    (e.g. ``convolution`` in ``Layer``); when ``base`` has no ``export_proto`` of its own
    the generated class exports the bare message.
    """
    field_names = [f.name for f in desc.fields]
    clash = set(field_names) & set(base_kwargs)
    if clash:
        raise RuntimeError(f"{desc.name}: fields {sorted(clash)} collide with base arguments")
    base_exports = hasattr(base, "export_proto")
    msg_cls = parent_message_cls

    def __init__(self, *args, **kwargs):
        own = {k: kwargs.pop(k) for k in list(kwargs) if k in field_names}
        unknown = [k for k in kwargs if k not in base_kwargs]
        if unknown:
            raise ValueError(f"{desc.name}: unknown argument(s) {unknown}")
        base.__init__(self, *args, **kwargs)
        for name in field_names:
            setattr(self, name, own.get(name))

    def export_proto(self):
        if base_exports:
            proto = base.export_proto(self)
            target = getattr(proto, parent_field)
            target.SetInParent()
        else:
            proto = msg_cls()
            target = proto
        set_message(target, **{n: getattr(self, n, None) for n in field_names})
        return proto

    doc = f"{desc.name}\n\nFields:\n" + ("".join(f"    {f.name}\n" for f in desc.fields) or "    none\n")
    ns = {"__init__": __init__, "export_proto": export_proto, "__doc__": doc,
          "get_field_names": lambda self: list(field_names), "_message_name": desc.name}
    for e in desc.enum_types:
        ns[e.name] = _enum_namespace(e)
    return type(desc.name, (base,), ns)


def classes_from_oneof(container_cls, base, base_kwargs, skip=(), bare=False):
    """One class per message-typed field of ``container_cls`` (skipping ``skip``)."""
    out = {}
    from google.protobuf import message_factory
    for f in container_cls.DESCRIPTOR.fields:
        if f.name in skip or f.message_type is None:
            continue
        if f.message_type.full_name.startswith("google.protobuf."):
            continue
        mcls = message_factory.GetMessageClass(f.message_type) if bare else None
        cls = class_from_message(f.message_type, f.name, base, base_kwargs, mcls)
        out[cls.__name__] = cls
    return out
