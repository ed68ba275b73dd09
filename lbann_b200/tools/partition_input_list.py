"""Shuffle a sample list ("<path> <label>" per line) and cut it into equal partitions.

Writes the shuffled list to ``<output>`` and partition ``p`` to ``<output>.p<p>``; lines
that do not fit an equal split are left out of the partitions, as in the reference tool
(tools/partition_input_list.cpp).
"""
from __future__ import annotations

import argparse
import random
from typing import List, Optional, Tuple


def read_list(path: str) -> List[Tuple[str, int]]:
    rows = []
    with open(path) as f:
        for line in f:
            line = line.rstrip("\n")
            if not line.strip():
                continue
            name, _, label = line.rpartition(" ")
            rows.append((name, int(label)))
    return rows


def partition(rows: List[Tuple[str, int]], num_partitions: int, seed: Optional[int] = None):
    if num_partitions < 1:
        raise ValueError("the number of partitions must be positive")
    rows = list(rows)
    random.Random(seed).shuffle(rows)
    per = len(rows) // num_partitions
    return rows, [rows[p * per:(p + 1) * per] for p in range(num_partitions)]


def write_list(path: str, rows) -> None:
    with open(path, "w") as f:
        for name, label in rows:
            f.write(f"{name} {label}\n")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("input_file")
    ap.add_argument("output_file_basename")
    ap.add_argument("num_partitions", type=int)
    ap.add_argument("--seed", type=int, default=None, help="default: a different shuffle every run")
    a = ap.parse_args(argv)
    rows = read_list(a.input_file)
    shuffled, parts = partition(rows, a.num_partitions, a.seed)
    print(f"A total of {len(rows)} rows  Num of partition {a.num_partitions}  "
          f"Data per partition {len(parts[0])}")
    write_list(a.output_file_basename, shuffled)
    for p, part in enumerate(parts):
        write_list(f"{a.output_file_basename}.p{p}", part)
        print(f"Partitioned file name {a.output_file_basename}.p{p}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
