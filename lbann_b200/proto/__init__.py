"""The ``lbann_data`` protobuf schema, built at import time from ``schema.py``.

``lbann_pb2`` style access: ``from lbann_b200.proto import lbann_pb2`` exposes every
message class of the package (``lbann_pb2.LbannPB``, ``lbann_pb2.Layer`` ...), and
``callbacks_pb2`` / ``layers_pb2`` ... alias the same namespace for code written against
the reference's generated modules (python/lbann/__init__.py imports them by those names).
"""
from __future__ import annotations

import types

from google.protobuf import any_pb2  # noqa: F401  (registers google.protobuf.Any)
from google.protobuf import wrappers_pb2  # noqa: F401
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

from . import schema
from ._dsl import EnumDef, FileDef, MessageDef

PACKAGE = "lbann_data"
_FDP = descriptor_pb2.FieldDescriptorProto
_SCALARS = {
    "double": _FDP.TYPE_DOUBLE, "float": _FDP.TYPE_FLOAT, "int32": _FDP.TYPE_INT32,
    "int64": _FDP.TYPE_INT64, "uint32": _FDP.TYPE_UINT32, "uint64": _FDP.TYPE_UINT64,
    "sint32": _FDP.TYPE_SINT32, "sint64": _FDP.TYPE_SINT64, "bool": _FDP.TYPE_BOOL,
    "string": _FDP.TYPE_STRING, "bytes": _FDP.TYPE_BYTES, "fixed32": _FDP.TYPE_FIXED32,
    "fixed64": _FDP.TYPE_FIXED64,
}


def _collect_symbols(files):
    """fully-qualified name -> 'message' | 'enum' for everything the tables define."""
    table = {}

    def walk_msg(prefix, m: MessageDef):
        fq = f"{prefix}.{m.name}"
        table[fq] = "message"
        for e in m.enums:
            table[f"{fq}.{e.name}"] = "enum"
        for n in m.nested:
            walk_msg(fq, n)

    for f in files:
        for e in f.enums:
            table[f"{PACKAGE}.{e.name}"] = "enum"
        for m in f.messages:
            walk_msg(PACKAGE, m)
    table["google.protobuf.Any"] = "message"
    for w in ("DoubleValue", "FloatValue", "Int64Value", "UInt64Value", "Int32Value",
              "UInt32Value", "BoolValue", "StringValue", "BytesValue"):
        table[f"google.protobuf.{w}"] = "message"
    return table


def _resolve(name: str, scope: str, symbols) -> str:
    if name.startswith("."):
        return name[1:]
    parts = scope.split(".")
    while True:
        cand = ".".join(parts + [name]) if parts else name
        if cand in symbols:
            return cand
        if not parts:
            raise KeyError(f"schema: cannot resolve type {name!r} from {scope!r}")
        parts.pop()


def _fill_enum(ep, e: EnumDef):
    ep.name = e.name
    for k, v in e.values:
        val = ep.value.add()
        val.name, val.number = k, v


def _camel(s: str) -> str:
    return "".join(p.capitalize() for p in s.split("_"))


def _fill_message(mp, m: MessageDef, scope: str, symbols):
    mp.name = m.name
    fq = f"{scope}.{m.name}"
    for e in m.enums:
        _fill_enum(mp.enum_type.add(), e)
    for n in m.nested:
        _fill_message(mp.nested_type.add(), n, fq, symbols)
    oneofs = []
    for f in m.fields:
        if f.oneof and f.oneof not in oneofs:
            oneofs.append(f.oneof)
            mp.oneof_decl.add().name = f.oneof
    for f in m.fields:
        fp = mp.field.add()
        fp.name, fp.number = f.name, f.number
        fp.json_name = f.name
        fp.label = _FDP.LABEL_REPEATED if f.repeated else _FDP.LABEL_OPTIONAL
        ftype = f.type
        if ftype.startswith("map<"):
            kt, vt = ftype[4:-1].split(",")
            entry = mp.nested_type.add()
            entry.name = _camel(f.name) + "Entry"
            entry.options.map_entry = True
            for idx, (nm, tp) in enumerate((("key", kt), ("value", vt)), start=1):
                ef = entry.field.add()
                ef.name, ef.number, ef.label = nm, idx, _FDP.LABEL_OPTIONAL
                ef.json_name = nm
                _set_type(ef, tp, fq, symbols)
            fp.label = _FDP.LABEL_REPEATED
            fp.type = _FDP.TYPE_MESSAGE
            fp.type_name = f".{fq}.{entry.name}"
            continue
        _set_type(fp, ftype, fq, symbols)
        if f.oneof:
            fp.oneof_index = oneofs.index(f.oneof)
        elif f.optional:
            # proto3 explicit presence = synthetic oneof
            mp.oneof_decl.add().name = f"_{f.name}"
            fp.oneof_index = len(mp.oneof_decl) - 1
            fp.proto3_optional = True


def _set_type(fp, ftype: str, scope: str, symbols):
    if ftype in _SCALARS:
        fp.type = _SCALARS[ftype]
        return
    fq = _resolve(ftype, scope, symbols)
    fp.type = _FDP.TYPE_ENUM if symbols[fq] == "enum" else _FDP.TYPE_MESSAGE
    fp.type_name = "." + fq


def _build():
    pool = descriptor_pool.Default()
    symbols = _collect_symbols(schema.FILES)
    # dependency order
    by_name = {f"{f.name}.proto": f for f in schema.FILES}
    files, seen = [], set()

    def visit(f):
        if f.name in seen:
            return
        seen.add(f.name)
        for imp in f.imports:
            if imp in by_name:
                visit(by_name[imp])
        files.append(f)

    for f in schema.FILES:
        visit(f)
    classes = {}
    enums = {}
    for f in files:
        fdp = descriptor_pb2.FileDescriptorProto()
        fdp.name = f"lbann_b200/{f.name}.proto"
        fdp.package = PACKAGE
        fdp.syntax = "proto3"
        for imp in f.imports:
            fdp.dependency.append(imp if imp.startswith("google/") else f"lbann_b200/{imp}")
        for e in f.enums:
            _fill_enum(fdp.enum_type.add(), e)
        for m in f.messages:
            _fill_message(fdp.message_type.add(), m, PACKAGE, symbols)
        pool.Add(fdp)
        fd = pool.FindFileByName(fdp.name)
        for name, md in fd.message_types_by_name.items():
            classes[name] = message_factory.GetMessageClass(md)
        for name, ed in fd.enum_types_by_name.items():
            enums[name] = ed
    return classes, enums


_classes, _enums = _build()


class _EnumWrapper:
    """Mimics the generated enum wrappers: ``DataType.FLOAT``, ``.Name()``, ``.Value()``."""

    def __init__(self, desc):
        self.DESCRIPTOR = desc
        for v in desc.values:
            setattr(self, v.name, v.number)

    def Name(self, number):
        return self.DESCRIPTOR.values_by_number[number].name

    def Value(self, name):
        return self.DESCRIPTOR.values_by_name[name].number

    def keys(self):
        return [v.name for v in self.DESCRIPTOR.values]


def _make_module(name: str) -> types.ModuleType:
    mod = types.ModuleType(name)
    for k, v in _classes.items():
        setattr(mod, k, v)
    for k, d in _enums.items():
        w = _EnumWrapper(d)
        setattr(mod, k, w)
        for val in d.values:
            setattr(mod, val.name, val.number)
    return mod


lbann_pb2 = _make_module("lbann_pb2")
for _n in ("callbacks", "layers", "metrics", "model", "objective_functions", "operators",
           "optimizers", "reader", "weights", "trainer", "training_algorithm", "datatype",
           "transforms", "data_coordinator"):
    globals()[f"{_n}_pb2"] = lbann_pb2


def message_class(name: str):
    """Message class by (possibly nested, dot-separated) name inside ``lbann_data``."""
    parts = name.split(".")
    cls = _classes[parts[0]]
    for p in parts[1:]:
        cls = getattr(cls, p)
    return cls


from . import serialize  # noqa: E402,F401
from .serialize import save_prototext  # noqa: E402,F401
