"""``python -m lbann.proto.bin2text in.protobin out.prototext``: a binary experiment (LbannPB)
in protobuf text format (python/lbann/proto/bin2text.py)."""
import sys

from google.protobuf import text_format

from . import lbann_pb2


def bin2text(infile: str, outfile: str) -> None:
    msg = lbann_pb2.LbannPB()
    with open(infile, "rb") as f:
        msg.ParseFromString(f.read())
    with open(outfile, "w") as f:
        f.write(text_format.MessageToString(msg, use_index_order=True))


if __name__ == "__main__":
    if len(sys.argv) != 3:
        raise SystemExit(__doc__)
    bin2text(sys.argv[1], sys.argv[2])
