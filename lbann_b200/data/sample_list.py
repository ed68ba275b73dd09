"""Sample lists: text files that name which samples of which bundle files form a data set.

Format (include/lbann/data_ingestion/readers/sample_list.hpp:42-110,
sample_list_impl.hpp:165-240, sample_list_open_files_impl.hpp:127-440)::

    <TYPE>                                   SINGLE-SAMPLE | MULTI-SAMPLE_INCLUSION[_V2] |
                                             MULTI-SAMPLE_EXCLUSION | CONDUIT_HDF5_INCLUSION |
                                             CONDUIT_HDF5_EXCLUSION
    <included> <excluded> <num files>        (SINGLE-SAMPLE: <num files>; *_V2: <included> <num files>)
    <data directory>
    [<label file>]                           (types with a label header line)
    <file> <included> <excluded> <id> ...    one line per bundle file; the ids are the included
                                             samples (inclusion) or the left-out ones (exclusion)
    <file> [<label>]                         SINGLE-SAMPLE

A list can be loaded with a stride and an offset (every rank of a trainer keeps lines
``offset, offset + stride, ...``), written back, and split into per-rank or per-trainer
lists.  Exclusion lists need the names of all samples of a bundle; ``names_of(path)``
provides them (for ``.npz`` bundles: the archive's top-level sample names).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

SINGLE = "SINGLE-SAMPLE"
INCLUSION = "MULTI-SAMPLE_INCLUSION"
INCLUSION_V2 = "MULTI-SAMPLE_INCLUSION_V2"
EXCLUSION = "MULTI-SAMPLE_EXCLUSION"
HDF5_INCLUSION = "CONDUIT_HDF5_INCLUSION"
HDF5_EXCLUSION = "CONDUIT_HDF5_EXCLUSION"


@dataclass
class SampleListHeader:
    kind: str = INCLUSION
    included: int = 0
    excluded: int = 0
    num_files: int = 0
    file_dir: str = ""
    label_file: str = ""

    @property
    def multi_sample(self) -> bool:
        return self.kind != SINGLE

    @property
    def exclusive(self) -> bool:
        return self.kind in (EXCLUSION, HDF5_EXCLUSION)

    @property
    def has_unused_fields(self) -> bool:
        return self.kind != INCLUSION_V2

    @property
    def has_label_line(self) -> bool:
        return self.kind in (SINGLE, INCLUSION, EXCLUSION)


def npz_sample_names(path: str) -> List[str]:
    """Sample names of an ``.npz`` bundle whose arrays are called ``<sample>/<field>``."""
    import numpy as np
    with np.load(path) as z:
        seen, out = set(), []
        for key in z.files:
            name = key.split("/", 1)[0]
            if name not in seen:
                seen.add(name)
                out.append(name)
    return out


@dataclass
class SampleList:
    header: SampleListHeader = field(default_factory=SampleListHeader)
    samples: List[Tuple[str, str]] = field(default_factory=list)    # (bundle file, sample name)
    labels: List[Optional[str]] = field(default_factory=list)        # SINGLE-SAMPLE label column

    # ------------------------------------------------------------------ reading
    @classmethod
    def load(cls, path: str, stride: int = 1, offset: int = 0,
             names_of: Optional[Callable[[str], Sequence[str]]] = None) -> "SampleList":
        with open(path) as f:
            return cls.load_from_string(f.read(), stride, offset, names_of, name=path)

    @classmethod
    def load_from_string(cls, text: str, stride: int = 1, offset: int = 0,
                         names_of: Optional[Callable[[str], Sequence[str]]] = None,
                         name: str = "<string>") -> "SampleList":
        lines = text.splitlines()
        if len(lines) < 3:
            raise ValueError(f"sample list {name}: the three header lines are missing")
        h = SampleListHeader()
        h.kind = lines[0].split()[0].upper() if lines[0].split() else ""
        if h.kind not in (SINGLE, INCLUSION, INCLUSION_V2, EXCLUSION, HDF5_INCLUSION, HDF5_EXCLUSION):
            raise ValueError(f"sample list {name}: unknown type '{lines[0].strip()}'")
        counts = [int(t) for t in lines[1].split()]
        try:
            if not h.multi_sample:
                h.num_files = counts[0]
                h.included = h.num_files
            elif h.has_unused_fields:
                h.included, h.excluded, h.num_files = counts[0], counts[1], counts[2]
            else:
                h.included, h.num_files = counts[0], counts[1]
        except IndexError:
            raise ValueError(f"sample list {name}: malformed count line '{lines[1]}'") from None
        h.file_dir = lines[2].split()[0] if lines[2].split() else ""
        if not h.file_dir:
            raise ValueError(f"sample list {name}: the data directory line is empty")
        body = 3
        if h.has_label_line and len(lines) > 3 and _looks_like_label_line(lines[3], h):
            h.label_file = lines[3].strip()
            body = 4
        out = cls(header=h)
        names_of = names_of or npz_sample_names
        nfile = 0
        for line in lines[body:]:
            tok = line.split()
            if not tok:
                continue
            if nfile >= h.num_files:
                break
            nfile += 1
            if (nfile - 1) % stride != offset:
                continue
            fname = tok[0]
            if not h.multi_sample:
                out.samples.append((fname, ""))
                out.labels.append(tok[1] if len(tok) > 1 else None)
                continue
            try:
                n_inc = int(tok[1])
                n_exc = int(tok[2]) if h.has_unused_fields else 0
            except (IndexError, ValueError):
                raise ValueError(f"sample list {name}: malformed line '{line}'") from None
            ids = tok[3:] if h.has_unused_fields else tok[2:]
            if h.exclusive:
                if len(ids) != n_exc:
                    raise ValueError(f"sample list {name}: '{fname}' lists {len(ids)} excluded "
                                     f"samples, its header says {n_exc}")
                left_out = set(ids)
                keep = [s for s in names_of(os.path.join(h.file_dir, fname)) if s not in left_out]
            else:
                if len(ids) != n_inc:
                    raise ValueError(f"sample list {name}: '{fname}' lists {len(ids)} samples, "
                                     f"its header says {n_inc}")
                keep = ids
            out.samples.extend((fname, s) for s in keep)
            out.labels.extend(None for _ in keep)
        return out

    # ------------------------------------------------------------------ queries
    def __len__(self):
        return len(self.samples)

    def files(self) -> List[str]:
        seen, out = set(), []
        for f, _ in self.samples:
            if f not in seen:
                seen.add(f)
                out.append(f)
        return out

    def path_of(self, index: int) -> str:
        return os.path.join(self.header.file_dir, self.samples[index][0])

    # ------------------------------------------------------------------ writing / splitting
    def to_string(self) -> str:
        """Always written as an inclusion list (every kept sample is named)."""
        h = self.header
        if not h.multi_sample:
            rows = [f"{f} {l}" if l is not None else f for (f, _), l in zip(self.samples, self.labels)]
            head = [SINGLE, str(len(rows)), h.file_dir]
            if h.label_file:
                head.append(h.label_file)
            return "\n".join(head + rows) + "\n"
        by_file = {}
        for f, s in self.samples:
            by_file.setdefault(f, []).append(s)
        rows = [f"{f} {len(ids)} 0 " + " ".join(ids) for f, ids in by_file.items()]
        head = [INCLUSION, f"{len(self.samples)} 0 {len(by_file)}", h.file_dir]
        if h.label_file:
            head.append(h.label_file)
        return "\n".join(head + rows) + "\n"

    def write(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_string())

    def partition(self, parts: int, keep_order: bool = True) -> List["SampleList"]:
        """Deal the samples into ``parts`` lists (per trainer or per rank): round-robin, or
        contiguous blocks when ``keep_order`` is off."""
        out = [SampleList(header=SampleListHeader(**vars(self.header))) for _ in range(parts)]
        n = len(self.samples)
        for i, (s, l) in enumerate(zip(self.samples, self.labels)):
            p = i % parts if keep_order else min(i * parts // max(n, 1), parts - 1)
            out[p].samples.append(s)
            out[p].labels.append(l)
        for o in out:
            o.header.included = len(o.samples)
            o.header.num_files = len(o.files())
        return out


def _looks_like_label_line(line: str, h: SampleListHeader) -> bool:
    """The optional fourth header line names a label / response file.  A body line starts
    with a bundle file name followed by counts (multi-sample) or has at most two tokens that
    name a data file (single-sample); a label line is one path that exists or ends in a
    label-file suffix."""
    tok = line.split()
    if len(tok) != 1:
        return False
    t = tok[0]
    return t.endswith((".csv", ".txt", ".labels", ".label", ".tsv")) and h.multi_sample
