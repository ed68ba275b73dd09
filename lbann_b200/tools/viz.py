"""``python -m lbann_b200.tools.viz model.prototext [graph.dot]``: the layer graph of an
experiment (or model) prototext as a Graphviz DOT file (scripts/viz.py of the reference, which
renders through the ``graphviz`` package; here the DOT text is written directly and any
Graphviz installation turns it into an image: ``dot -Tpdf graph.dot -o graph.pdf``).

Nodes are coloured by sub-grid (``grid_tag``), edges that cross sub-grids can be highlighted,
layers with a parallel strategy get a double border.
"""
from __future__ import annotations

import argparse

from google.protobuf import text_format

PALETTE = ["#ffffff", "#a0c4ff", "#ffadad", "#fdffb6", "#caffbf", "#9bf6ff", "#bdb2ff", "#ffc6ff", "#ffd6a5"]


def load_model(path: str):
    from ..proto import lbann_pb2
    text = open(path).read()
    exp = lbann_pb2.LbannPB()
    try:
        text_format.Parse(text, exp)
        if len(exp.model.layer):
            return exp.model
    except text_format.ParseError:
        pass
    model = lbann_pb2.Model()
    text_format.Parse(text, model)
    return model


def layer_type(layer) -> str:
    return layer.WhichOneof("layer_type") or "layer"


def to_dot(model, label_format: str = "type-only", color_cross_grid: bool = False) -> str:
    tag = {l.name: (l.grid_tag.value if l.HasField("grid_tag") else 0) for l in model.layer}
    lines = ["digraph model {", "  rankdir=TB;", '  node [shape=box, style="rounded,filled", fontname="Helvetica"];']
    for l in model.layer:
        t = layer_type(l)
        if label_format == "type-only":
            label = t
        elif label_format == "name-only":
            label = l.name
        elif label_format == "type-and-name":
            label = f"{t}\\n{l.name}"
        else:
            fields = text_format.MessageToString(getattr(l, t), as_one_line=True) if t != "layer" else ""
            label = f"{t}\\n{l.name}" + (f"\\n{fields[:80]}" if fields else "")
        color = PALETTE[tag[l.name] % len(PALETTE)]
        extra = ", peripheries=2" if l.HasField("parallel_strategy") else ""
        lines.append(f'  "{l.name}" [label="{label}", fillcolor="{color}"{extra}];')
    for l in model.layer:
        for p in l.parents:
            attrs = ""
            if color_cross_grid and tag.get(p, 0) != tag[l.name]:
                attrs = ' [color="red", penwidth=2]'
            lines.append(f'  "{p}" -> "{l.name}"{attrs};')
    lines.append("}")
    return "\n".join(lines) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Write an LBANN model's layer graph as a Graphviz DOT file.")
    ap.add_argument("input", help="experiment or model prototext file")
    ap.add_argument("output", nargs="?", default="graph.dot")
    ap.add_argument("--label-format", default="type-only", choices=("type-only", "name-only", "type-and-name", "full"))
    ap.add_argument("--color-cross-grid", action="store_true", help="highlight edges between sub-grids")
    a = ap.parse_args(argv)
    with open(a.output, "w") as f:
        f.write(to_dot(load_model(a.input), a.label_format, a.color_cross_grid))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
