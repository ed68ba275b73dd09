"""``python -m lbann.proto.text2bin in.prototext out.protobin``: a text-format experiment
(LbannPB) as a binary protobuf (python/lbann/proto/text2bin.py)."""
import sys

from google.protobuf import text_format

from . import lbann_pb2


def text2bin(infile: str, outfile: str) -> None:
    msg = lbann_pb2.LbannPB()
    with open(infile) as f:
        text_format.Parse(f.read(), msg)
    with open(outfile, "wb") as f:
        f.write(msg.SerializeToString())


if __name__ == "__main__":
    if len(sys.argv) != 3:
        raise SystemExit(__doc__)
    text2bin(sys.argv[1], sys.argv[2])
