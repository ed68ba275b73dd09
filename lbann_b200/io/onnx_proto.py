"""The subset of the ONNX protobuf schema that a model export needs (ModelProto, GraphProto,
NodeProto, AttributeProto, TensorProto, ValueInfoProto, TypeProto, TensorShapeProto,
OperatorSetIdProto), declared with the field numbers of the public ``onnx.proto`` so that
the files written here load in any ONNX consumer.  The ``onnx`` Python package is not needed.
"""
from __future__ import annotations

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_F = descriptor_pb2.FieldDescriptorProto
_T = {"int64": _F.TYPE_INT64, "int32": _F.TYPE_INT32, "float": _F.TYPE_FLOAT, "double": _F.TYPE_DOUBLE,
      "string": _F.TYPE_STRING, "bytes": _F.TYPE_BYTES, "uint64": _F.TYPE_UINT64}

# message -> [(field, number, type, repeated)]; a type that is not a scalar names a message
_SCHEMA = {
    "OperatorSetIdProto": [("domain", 1, "string", False), ("version", 2, "int64", False)],
    "StringStringEntryProto": [("key", 1, "string", False), ("value", 2, "string", False)],
    "TensorProto": [("dims", 1, "int64", True), ("data_type", 2, "int32", False),
                    ("float_data", 4, "float", True), ("int32_data", 5, "int32", True),
                    ("string_data", 6, "bytes", True), ("int64_data", 7, "int64", True),
                    ("name", 8, "string", False), ("raw_data", 9, "bytes", False),
                    ("double_data", 10, "double", True), ("uint64_data", 11, "uint64", True),
                    ("doc_string", 12, "string", False)],
    "TensorShapeProto.Dimension": [("dim_value", 1, "int64", False), ("dim_param", 2, "string", False),
                                   ("denotation", 3, "string", False)],
    "TensorShapeProto": [("dim", 1, "TensorShapeProto.Dimension", True)],
    "TypeProto.Tensor": [("elem_type", 1, "int32", False), ("shape", 2, "TensorShapeProto", False)],
    "TypeProto": [("tensor_type", 1, "TypeProto.Tensor", False), ("denotation", 6, "string", False)],
    "ValueInfoProto": [("name", 1, "string", False), ("type", 2, "TypeProto", False),
                       ("doc_string", 3, "string", False)],
    "AttributeProto": [("name", 1, "string", False), ("f", 2, "float", False), ("i", 3, "int64", False),
                       ("s", 4, "bytes", False), ("t", 5, "TensorProto", False),
                       ("floats", 7, "float", True), ("ints", 8, "int64", True), ("strings", 9, "bytes", True),
                       ("doc_string", 13, "string", False), ("type", 20, "int32", False)],
    "NodeProto": [("input", 1, "string", True), ("output", 2, "string", True), ("name", 3, "string", False),
                  ("op_type", 4, "string", False), ("attribute", 5, "AttributeProto", True),
                  ("doc_string", 6, "string", False), ("domain", 7, "string", False)],
    "GraphProto": [("node", 1, "NodeProto", True), ("name", 2, "string", False),
                   ("initializer", 5, "TensorProto", True), ("doc_string", 10, "string", False),
                   ("input", 11, "ValueInfoProto", True), ("output", 12, "ValueInfoProto", True),
                   ("value_info", 13, "ValueInfoProto", True)],
    "ModelProto": [("ir_version", 1, "int64", False), ("producer_name", 2, "string", False),
                   ("producer_version", 3, "string", False), ("domain", 4, "string", False),
                   ("model_version", 5, "int64", False), ("doc_string", 6, "string", False),
                   ("graph", 7, "GraphProto", False), ("opset_import", 8, "OperatorSetIdProto", True),
                   ("metadata_props", 14, "StringStringEntryProto", True)],
}

# TensorProto.DataType / AttributeProto.AttributeType values used by the exporter
FLOAT, INT64, FLOAT16, BFLOAT16 = 1, 7, 10, 16
ATTR_FLOAT, ATTR_INT, ATTR_STRING, ATTR_TENSOR, ATTR_FLOATS, ATTR_INTS = 1, 2, 3, 4, 6, 7


def _build():
    fd = descriptor_pb2.FileDescriptorProto()
    fd.name, fd.package, fd.syntax = "lbann_b200_onnx_subset.proto", "onnx", "proto3"
    top = {}
    for full in _SCHEMA:                     # parents are declared before their nested messages are filled
        parts = full.split(".")
        if len(parts) == 1:
            mp = fd.message_type.add()
            mp.name = full
            top[full] = mp
    for full in _SCHEMA:
        parts = full.split(".")
        if len(parts) == 2:
            mp = top[parts[0]].nested_type.add()
            mp.name = parts[1]
            top[full] = mp
    for full, fields in _SCHEMA.items():
        mp = top[full]
        for name, number, ftype, repeated in fields:
            fp = mp.field.add()
            fp.name, fp.number, fp.json_name = name, number, name
            fp.label = _F.LABEL_REPEATED if repeated else _F.LABEL_OPTIONAL
            if ftype in _T:
                fp.type = _T[ftype]
            else:
                fp.type, fp.type_name = _F.TYPE_MESSAGE, f".onnx.{ftype}"
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    get = getattr(message_factory, "GetMessageClass", None)
    out = {}
    for full in _SCHEMA:
        desc = pool.FindMessageTypeByName(f"onnx.{full}")
        out[full] = get(desc) if get else message_factory.MessageFactory(pool).GetPrototype(desc)
    return out


_CLASSES = _build()
ModelProto = _CLASSES["ModelProto"]
GraphProto = _CLASSES["GraphProto"]
NodeProto = _CLASSES["NodeProto"]
TensorProto = _CLASSES["TensorProto"]
ValueInfoProto = _CLASSES["ValueInfoProto"]
AttributeProto = _CLASSES["AttributeProto"]
