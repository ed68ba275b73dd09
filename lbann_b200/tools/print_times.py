"""``python -m lbann_b200.tools.print_times run.log [--csv out.csv]``: the per-epoch numbers
that the ``print_statistics`` and ``timer`` callbacks write to standard output, as a table
(scripts/plotting/print_times.py of the reference reads the same lines).

Recognised lines (the formats of src/callbacks/print_statistics.cpp and timer.cpp):

    model0 (instance 0) training epoch 3 objective function : 0.123
    model0 (instance 0) training epoch 3 accuracy : 98.1%
    model0 (instance 0) training epoch 3 run time : 12.3s
    model0 (instance 0) training epoch 3 mini-batch time statistics : 0.01s mean, ...
"""
from __future__ import annotations

import argparse
import csv
import re
import sys
from collections import OrderedDict

LINE = re.compile(r"^(?P<model>\S+) \(instance (?P<inst>\d+)\) (?P<mode>training|validation|test) "
                  r"(?:epoch (?P<epoch>\d+) )?(?P<what>[^:]+?) : (?P<value>.+)$")
NUMBER = re.compile(r"[-+]?(?:\d+\.?\d*|\.\d+)(?:[eE][-+]?\d+)?")


def parse(lines):
    """[(model, mode, epoch, quantity, value)] for every recognised line."""
    rows = []
    for line in lines:
        m = LINE.match(line.strip())
        if not m:
            continue
        num = NUMBER.search(m.group("value"))
        if not num:
            continue
        epoch = int(m.group("epoch")) if m.group("epoch") is not None else -1
        rows.append((m.group("model"), m.group("mode"), epoch, m.group("what").strip(), float(num.group(0))))
    return rows


def table(rows):
    """{(model, mode, epoch): {quantity: value}} in order of appearance."""
    out = OrderedDict()
    for model, mode, epoch, what, value in rows:
        out.setdefault((model, mode, epoch), OrderedDict())[what] = value
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Per-epoch statistics of a training log as a table.")
    ap.add_argument("log")
    ap.add_argument("--csv", help="also write the table to this file")
    a = ap.parse_args(argv)
    with open(a.log) as f:
        tab = table(parse(f))
    cols = []
    for vals in tab.values():
        for k in vals:
            if k not in cols:
                cols.append(k)
    header = ["model", "mode", "epoch"] + cols
    data = [[k[0], k[1], k[2]] + [v.get(c, "") for c in cols] for k, v in tab.items()]
    widths = [max(len(str(x)) for x in [h] + [r[i] for r in data]) for i, h in enumerate(header)]
    for r in [header] + data:
        print("  ".join(str(x).ljust(w) for x, w in zip(r, widths)))
    if a.csv:
        with open(a.csv, "w", newline="") as f:
            csv.writer(f).writerows([header] + data)
    return 0


if __name__ == "__main__":
    sys.exit(main())
