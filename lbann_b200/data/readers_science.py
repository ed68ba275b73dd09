"""Readers of the reference's application data sets: NCI (delimited text), mesh (one raw
float32 file per channel and sample), Pilot-2 molecular frames and RAS lipid frames (``.npz``),
JAG simulation bundles.  The reference reads the last two through Conduit / HDF5; here a
bundle is an ``.npz`` archive (see ``SampleListReader``), the fields and their meaning are the
reference's.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np

from .readers import CsvReader, DataReader, SampleListReader, register


@register("nci")
class NciReader(CsvReader):
    """NCI drug-response table: space separated, one broken header row, five metadata columns
    in front of the features; column 2 is the response, column 3 the class ("rs" -> 0,
    anything else -> 1) (src/data_ingestion/readers/data_reader_nci.cpp:38-52)."""

    META_COLS, RESPONSE_COL, LABEL_COL = 5, 2, 3

    def load(self):
        p = self.proto
        path = os.path.join(p.data_filedir, p.data_filename)
        feats, resp, labels = [], [], []
        with open(path) as f:
            next(f, None)                                  # the header row is not usable
            for line in f:
                tok = line.split()
                if len(tok) <= self.META_COLS:
                    continue
                resp.append(float(tok[self.RESPONSE_COL]))
                labels.append(0 if tok[self.LABEL_COL] == "rs" else 1)
                feats.append([float(v) for v in tok[self.META_COLS:]])
        self.arr = np.asarray(feats, dtype=np.float32)
        self.resp = np.asarray(resp, dtype=np.float32)
        self.labels = np.asarray(labels, dtype=np.int64)
        self.num_labels = self.num_labels or 2
        self._fields = {"samples": (self.arr.shape[1],), "labels": (self.num_labels,), "responses": (1,)}

    def total_samples(self):
        return self.arr.shape[0]

    def fetch_field(self, field, index):
        if field == "samples":
            return self.arr[index]
        if field == "labels":
            return self.one_hot(int(self.labels[index]))
        return self.resp[index:index + 1]


@register("mesh")
class MeshReader(DataReader):
    """Unstructured-mesh quality images: for every sample one raw float32 file per channel,
    ``<dir>/<channel><suffix>/<channel><zero-padded index>.bin`` holding height rows of width
    values; the sample stacks the channels, the response is the ``mask`` channel.
    Random horizontal / vertical flips apply to all channels and the target of a sample alike
    (src/data_ingestion/readers/data_reader_mesh.cpp:41-176; defaults from data_reader_mesh.hpp:101-141)."""

    channels: Sequence[str] = ("Density", "Vorticity", "VelocityMagnitude", "Pressure", "SoundSpeed",
                               "ArtificialViscosity", "DivV", "Volume", "MeshQuality", "Energy",
                               "Temperature", "MaxShearStrainRate", "PlasticStrain")
    target, suffix, index_length = "mask", "128", 4
    height = width = 128
    random_flips = False

    def load(self):
        p = self.proto
        self.dir = p.data_filedir if p.data_filedir.endswith("/") or not p.data_filedir else p.data_filedir + "/"
        fmt = (getattr(p, "format", "") or "").split()
        # "format" may carry: suffix=<s> height=<h> width=<w> index_length=<n> flips channels=a,b,c
        for tok in fmt:
            k, _, v = tok.partition("=")
            if k == "suffix":
                self.suffix = v
            elif k == "height":
                self.height = int(v)
            elif k == "width":
                self.width = int(v)
            elif k == "index_length":
                self.index_length = int(v)
            elif k == "flips":
                self.random_flips = True
            elif k == "channels":
                self.channels = tuple(v.split(","))
            elif k == "target":
                self.target = v
        if self.height <= 0 or self.width <= 0:
            raise ValueError("mesh reader: data shape must be non-zero")
        found = glob.glob(f"{self.dir}{self.target}{self.suffix}/*.bin")
        if not found:
            raise ValueError("mesh reader: could not find any targets")
        self.n = len(found)
        if 10 ** self.index_length <= self.n:
            raise ValueError("mesh reader: index length too small")
        self._fields = {"samples": (len(self.channels), self.height, self.width),
                        "responses": (self.height, self.width)}
        self._flips: Dict[int, Tuple[int, int]] = {}
        self._rng = np.random.RandomState(1234)

    def total_samples(self):
        return self.n

    def _file(self, channel: str, index: int) -> str:
        return f"{self.dir}{channel}{self.suffix}/{channel}{index:0{self.index_length}d}.bin"

    def _load(self, channel: str, index: int) -> np.ndarray:
        a = np.fromfile(self._file(channel, index), dtype=np.float32, count=self.height * self.width)
        if a.size != self.height * self.width:
            raise ValueError(f"mesh reader: failed to read {self._file(channel, index)}")
        a = a.reshape(self.height, self.width)          # files hold `height` rows of `width` values
        fh, fv = self._flips.get(index, (0, 0))
        if fh:
            a = a[:, ::-1]
        if fv:
            a = a[::-1, :]
        return np.ascontiguousarray(a)

    def fetch_field(self, field, index):
        if field == "samples":
            if self.random_flips:                          # drawn per fetch of the sample, reused by its target
                self._flips[index] = (int(self._rng.randint(2)), int(self._rng.randint(2)))
            return np.stack([self._load(c, index) for c in self.channels])
        return self._load(self.target, index)


@register("pilot2_molecular_reader", "pilot2_molecular")
class Pilot2MolecularReader(DataReader):
    """Pilot-2 lipid simulation frames: ``features`` [frames, molecules, beads, 20] and
    ``neighbors`` [frames, molecules, 2 * max_neighborhood] in one ``.npz``.  A sample is a
    molecule of a frame followed by its first ``num_neighbors`` neighbours (zeros where the
    neighbour id is -1); positions (features 0-2) are divided by 320, bond lengths (8-19) by 10
    (src/data_ingestion/readers/data_reader_pilot2_molecular.cpp:47-199,
    include/.../data_reader_pilot2_molecular.hpp:70-86, 140-141)."""

    position_scale, bond_scale = 320.0, 10.0

    def load(self):
        p = self.proto
        z = np.load(os.path.join(p.data_filedir, p.data_filename))
        if "features" not in z.files:
            raise ValueError("pilot2_molecular: no features")
        if "neighbors" not in z.files:
            raise ValueError("pilot2_molecular: no neighbors")
        self.features = np.asarray(z["features"])
        self.neighbors = np.asarray(z["neighbors"])
        if self.features.ndim != 4:
            raise ValueError("pilot2_molecular: features must be [frames, molecules, beads, values]")
        self.num_neighbors = int(p.num_neighbors)
        self.max_neighborhood = int(p.max_neighborhood) or self.neighbors.shape[-1] // 2
        self.per_frame = self.features.shape[1]
        nb, nv = self.features.shape[2], self.features.shape[3]
        scale = np.ones(nv, dtype=np.float32)
        idx = np.arange(nv) % 20
        scale[idx <= 2] = 1.0 / self.position_scale
        scale[(idx >= 8) & (idx <= 19)] = 1.0 / self.bond_scale
        self.scale = scale
        self._fields = {"samples": (self.num_neighbors + 1, nb, nv)}

    def total_samples(self):
        return self.features.shape[0] * self.per_frame

    def fetch_field(self, field, index):
        frame, mol = divmod(index, self.per_frame)
        out = np.zeros(self._fields["samples"], dtype=np.float32)
        out[0] = self.features[frame, mol] * self.scale
        nbrs = self.neighbors[frame, mol].reshape(-1)
        for i in range(1, self.num_neighbors + 1):
            j = int(nbrs[i]) if i < nbrs.size else -1
            if j != -1:
                out[i] = self.features[frame, j] * self.scale
        return out


@register("ras_lipid", "npz_ras_lipid")
class RasLipidReader(DataReader):
    """RAS-membrane simulation frames, one ``.npz`` per trajectory piece with the arrays
    ``density_sig1`` [frames, 13, 13, 14] (lipid densities, the sample), ``states`` [frames]
    (the label, 3 classes), ``bbs`` [frames, 184, 3] and ``probs`` [frames, 3].  ``seq_len``
    consecutive frames of one file form a sample (label = state of the last frame); the
    densities are normalised per channel from a table of ``max min mean std`` rows, as min-max
    or, with ``z_score``, as z-scores
    (src/data_ingestion/readers/data_reader_npz_ras_lipid.cpp:110-200, 217-232, 519-560)."""

    def load(self):
        p = self.proto
        pattern = os.path.join(p.data_filedir, p.data_file_pattern or p.data_filename or "*.npz")
        self.files = sorted(glob.glob(pattern))
        if not self.files:
            raise ValueError(f"ras_lipid: no files match {pattern}")
        opts = dict(tok.partition("=")[::2] for tok in (getattr(p, "format", "") or "").split())
        self.seq_len = int(opts.get("seq_len", 1) or 1)
        self.z_score = opts.get("z_score", "0") not in ("0", "", "false")
        self._z: Dict[int, object] = {}
        self.index: List[Tuple[int, int]] = []           # (file, first frame) of every sample
        dshape = None
        for fi, path in enumerate(self.files[:int(p.max_files_to_load) or None]):
            z = np.load(path)
            n = int(z["states"].shape[0]) // self.seq_len
            self.index += [(fi, k * self.seq_len) for k in range(n)]
            dshape = dshape or tuple(z["density_sig1"].shape[1:])
        self.num_labels = self.num_labels or 3
        self._fields = {"samples": (self.seq_len,) + dshape, "labels": (self.num_labels,),
                        "bbs": (self.seq_len, 184, 3), "probs": (self.seq_len, 3)}
        self.norm = None
        if p.metadata_filename:
            t = np.loadtxt(os.path.join(p.data_filedir, p.metadata_filename), ndmin=2)   # max min mean std
            if t.shape[0] != dshape[-1]:
                raise ValueError(f"normalization.size() = {t.shape[0]}; should be {dshape[-1]}")
            self.norm = t.astype(np.float32)

    def total_samples(self):
        return len(self.index)

    def _open(self, fi):
        z = self._z.get(fi)
        if z is None:
            if len(self._z) >= 8:
                self._z.pop(next(iter(self._z))).close()
            z = self._z[fi] = np.load(self.files[fi])
        return z

    def fetch_field(self, field, index):
        fi, f0 = self.index[index]
        z = self._open(fi)
        sl = slice(f0, f0 + self.seq_len)
        if field == "labels":
            return self.one_hot(int(z["states"][f0 + self.seq_len - 1]))
        if field == "samples":
            d = np.asarray(z["density_sig1"][sl], dtype=np.float32)
            if self.norm is not None:
                mx, mn, mean, std = (self.norm[:, i] for i in range(4))
                d = (d - mean) / std if self.z_score else (d - mn) / (mx - mn)
            return d
        return np.asarray(z[field][sl], dtype=np.float32).reshape(self._fields[field])


@register("jag_conduit", "jag")
class JagReader(SampleListReader):
    """JAG inertial-confinement-fusion bundles through a sample list.  Every sample holds
    ``inputs/<key>`` (5 simulation parameters), ``scalars/<key>`` (15+ diagnostics) and
    ``images/<key>`` (X-ray views).  The ``DataSetMetaData.Schema`` of the experiment names
    the keys to use and which kinds form the independent variable (data field ``samples``) and
    the dependent one (``responses``); ``Normalization`` gives one (scale, bias) per key
    (src/data_ingestion/readers/data_reader_jag_conduit.cpp:556-700, 1180-1330;
    src/proto/data_set_metadata.proto)."""

    KINDS = {1: "images", 2: "scalars", 3: "inputs"}

    def __init__(self, proto=None, role="train", metadata=None, **kw):
        super().__init__(proto, role=role, **kw)
        self.metadata = metadata

    def load(self):
        super().load()
        md = self.metadata
        sch = md.schema if md is not None else None
        name = self.sample_list.samples[0][1]
        first = self._bundle(0)
        have: Dict[str, List[str]] = {"images": [], "scalars": [], "inputs": []}
        for key in first.files:
            parts = key.split("/")
            if len(parts) == 3 and parts[0] == name and parts[1] in have:
                have[parts[1]].append(parts[2])
        pick = {
            "images": list(sch.jag_image_keys) if sch is not None and len(sch.jag_image_keys) else sorted(have["images"]),
            "scalars": list(sch.jag_scalar_keys) if sch is not None and len(sch.jag_scalar_keys) else sorted(have["scalars"]),
            "inputs": list(sch.jag_input_keys) if sch is not None and len(sch.jag_input_keys) else sorted(have["inputs"]),
        }
        for kind, keys in pick.items():
            missing = [k for k in keys if k not in have[kind]]
            if missing:
                raise ValueError(f"jag reader: {kind} keys {missing} are not in the bundles")
        self.keys = pick
        norm = md.normalization if md is not None else None
        table = {"images": getattr(norm, "jag_image_normalization_params", []),
                 "scalars": getattr(norm, "jag_scalar_normalization_params", []),
                 "inputs": getattr(norm, "jag_input_normalization_params", [])}
        self.affine = {}
        for kind, keys in pick.items():
            prm = list(table[kind])
            if prm and len(prm) != len(keys):
                raise ValueError(f"jag reader: {len(prm)} normalization entries for {len(keys)} {kind}")
            self.affine[kind] = [(float(q.scale), float(q.bias)) for q in prm] or [(1.0, 0.0)] * len(keys)

        def kinds(slices, default):
            out = [self.KINDS[int(v)] for s in slices for v in s.pieces if int(v) in self.KINDS]
            return out or default
        self.independent = kinds(sch.independent if sch is not None else [], ["images"] if pick["images"] else ["scalars"])
        self.dependent = kinds(sch.dependent if sch is not None else [], ["inputs"])
        self._sizes = {kind: [int(np.asarray(first[f"{name}/{kind}/{k}"]).size) for k in keys]
                       for kind, keys in pick.items()}
        self._fields = {"samples": (sum(sum(self._sizes[k]) for k in self.independent),),
                        "responses": (sum(sum(self._sizes[k]) for k in self.dependent),)}

    def slice_points(self, which: str) -> List[int]:
        """Offsets of the pieces of the independent / dependent variable, for a slice layer."""
        kinds = self.independent if which.startswith("ind") else self.dependent
        pts = [0]
        for k in kinds:
            pts.append(pts[-1] + sum(self._sizes[k]))
        return pts

    def _gather(self, index, kinds):
        z = self._bundle(index)
        name = self.sample_list.samples[index][1]
        out = []
        for kind in kinds:
            for key, (scale, bias) in zip(self.keys[kind], self.affine[kind]):
                a = np.asarray(z[f"{name}/{kind}/{key}"], dtype=np.float32).reshape(-1)
                out.append(a * scale + bias)
        return np.concatenate(out) if out else np.zeros(0, dtype=np.float32)

    def fetch_field(self, field, index):
        return self._gather(index, self.independent if field == "samples" else self.dependent)
