"""Write / read experiment files (python/lbann/proto/serialize.py:8-52 of the reference)."""
from __future__ import annotations

from google.protobuf import message as _pbmsg
from google.protobuf import text_format

from . import lbann_pb2


def build_experiment(**kwargs):
    """LbannPB from ``trainer=``, ``model=``, ``data_reader=``, ``optimizer=`` ... objects
    (front-end objects with ``export_proto`` or protobuf messages)."""
    msg = lbann_pb2.LbannPB()
    names = msg.DESCRIPTOR.fields_by_name.keys()
    for key, val in kwargs.items():
        if key not in names:
            raise TypeError(f"'{key}' is an invalid keyword argument for this function")
        if val is None:
            continue
        field = getattr(msg, key)
        field.CopyFrom(val if isinstance(val, _pbmsg.Message) else val.export_proto())
        field.SetInParent()
    if not msg.HasField("optimizer"):
        msg.optimizer.no_optimizer.SetInParent()
    return msg


def save_prototext(filename, binary=False, **kwargs):
    msg = build_experiment(**kwargs)
    with open(filename, "wb") as f:
        if binary:
            f.write(msg.SerializeToString())
        else:
            f.write(text_format.MessageToString(msg, use_index_order=True).encode())
    return msg


def text2bin(infile: str, outfile: str):
    msg = lbann_pb2.LbannPB()
    with open(infile, "rb") as f:
        text_format.Parse(f.read().decode(), msg)
    with open(outfile, "wb") as f:
        f.write(msg.SerializeToString())


def bin2text(infile: str, outfile: str):
    msg = lbann_pb2.LbannPB()
    with open(infile, "rb") as f:
        msg.ParseFromString(f.read())
    with open(outfile, "wb") as f:
        f.write(text_format.MessageToString(msg, use_index_order=True).encode())
