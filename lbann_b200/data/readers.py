"""Data readers.

A reader exposes named fields (``samples``, ``labels``, ``responses`` or arbitrary names)
with fixed per-sample dims and fetches samples by index into CPU tensors.  Index shuffling,
``fraction_of_data_to_use`` / ``first_n`` / ``absolute_sample_count`` and the validation /
tournament split follow ``generic_data_reader`` (src/data_ingestion/data_reader.cpp); the
concrete readers mirror src/data_ingestion/readers/*.cpp as noted per class.
"""
from __future__ import annotations

import gzip
import importlib
import math
import os
import pickle
import struct
import sys
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

READER_REGISTRY: Dict[str, type] = {}


def register(*names):
    def deco(cls):
        for n in names:
            READER_REGISTRY[n] = cls
        return cls
    return deco


def _ints(s) -> Tuple[int, ...]:
    if isinstance(s, str):
        return tuple(int(v) for v in s.replace(",", " ").split())
    return tuple(int(v) for v in s)


class DataReader:
    """Base reader.  Subclasses implement ``load()`` (discover the data set) and
    ``fetch_field(field, index) -> np.ndarray``."""

    def __init__(self, proto=None, role: str = "train", **kw):
        self.proto = proto
        self.name = getattr(proto, "name", kw.get("name", "reader"))
        self.role = role
        self.shuffle = bool(getattr(proto, "shuffle", kw.get("shuffle", False)))
        self.fraction = float(getattr(proto, "fraction_of_data_to_use", 0.0) or kw.get("fraction", 1.0))
        self.first_n = int(getattr(proto, "first_n", 0) or 0)
        self.absolute_count = int(getattr(proto, "absolute_sample_count", 0) or 0)
        self.validation_fraction = float(getattr(proto, "validation_fraction", 0.0) or 0.0)
        self.tournament_fraction = float(getattr(proto, "tournament_fraction", 0.0) or 0.0)
        self.num_labels = int(getattr(proto, "num_labels", 0) or kw.get("num_labels", 0))
        self.transforms = None
        self.indices: np.ndarray = np.zeros(0, dtype=np.int64)
        self._fields: Dict[str, Tuple[int, ...]] = {}

    # ---- to implement
    def load(self):
        raise NotImplementedError

    def fetch_field(self, field: str, index: int) -> np.ndarray:
        raise NotImplementedError

    def total_samples(self) -> int:
        raise NotImplementedError

    # ---- generic behaviour
    def fields(self) -> Dict[str, Tuple[int, ...]]:
        return self._fields

    def dims(self, field: str) -> Tuple[int, ...]:
        if field not in self._fields:
            raise KeyError(f"reader '{self.name}' ({self.role}) has no data field '{field}'; "
                           f"available: {sorted(self._fields)}")
        return self._fields[field]

    def setup(self, seed: int = 0):
        self.load()
        n = self.total_samples()
        idx = np.arange(n, dtype=np.int64)
        rng = np.random.RandomState((seed * 9973 + 12345) % (2 ** 31 - 1))
        if self.shuffle and not self.first_n:
            rng.shuffle(idx)
        if self.first_n:
            idx = idx[:self.first_n]
        elif self.absolute_count:
            idx = idx[:self.absolute_count]
        elif 0.0 < self.fraction < 1.0:
            idx = idx[:max(1, int(math.ceil(self.fraction * n)))]
        self.indices = idx
        return self

    def split(self, fraction: float):
        """Carve the trailing ``fraction`` of the index list out as a new index array."""
        n = len(self.indices)
        k = int(fraction * n + 0.5)
        if k <= 0:
            return np.zeros(0, dtype=np.int64)
        part, self.indices = self.indices[n - k:], self.indices[:n - k]
        return part

    def num_samples(self) -> int:
        return len(self.indices)

    def fetch_batch(self, idx: Sequence[int], fields: Sequence[str]) -> Dict[str, torch.Tensor]:
        out = {}
        for f in fields:
            arrs = [np.asarray(self.fetch_field(f, int(i))) for i in idx]
            if self.transforms is not None and f == "samples":
                arrs = [self.transforms(a) for a in arrs]
            a = np.stack(arrs) if arrs else np.zeros((0,) + self.dims(f), dtype=np.float32)
            t = torch.from_numpy(np.ascontiguousarray(a))
            if t.is_floating_point() and t.dtype != torch.float32:
                t = t.float()
            out[f] = t.reshape(len(idx), *self.dims(f))
        return out

    def one_hot(self, label: int) -> np.ndarray:
        v = np.zeros(self.num_labels, dtype=np.float32)
        if 0 <= label < self.num_labels:
            v[label] = 1.0
        return v

    def slice_points(self, which: str) -> List[int]:
        raise NotImplementedError(f"reader '{self.name}' provides no slice points")

    def state(self):
        return {"indices": self.indices.copy()}

    def load_state(self, st):
        self.indices = np.asarray(st["indices"], dtype=np.int64)


@register("synthetic")
class SyntheticReader(DataReader):
    """Random samples of a given shape (src/data_ingestion/readers/data_reader_synthetic.cpp:
    38-165): N(0,1) samples, uniform one-hot labels, N(0,1) responses.  Extensions:
    ``synth_distribution`` in {normal, uniform, lognormal, uniform_pm1, randint:<K>} selects
    the sample distribution (responses use uniform_pm1 when it is set on them via
    ``name:dist`` pairs, e.g. ``"samples:lognormal responses:uniform_pm1"``), and
    ``synth_pool_size`` pre-generates that many samples and cycles through them."""

    def load(self):
        p = self.proto
        self.n = int(getattr(p, "num_samples", 0) or 0)
        sd = _ints(getattr(p, "synth_dimensions", "") or "1")
        self._fields = {"samples": sd}
        if self.num_labels:
            self._fields["labels"] = (self.num_labels,)
        rd = getattr(p, "synth_response_dimensions", "")
        if rd:
            self._fields["responses"] = _ints(rd)
        self.dist = {"samples": "normal", "responses": "normal"}
        spec = getattr(p, "synth_distribution", "") or ""
        for tok in spec.split():
            if ":" in tok and not tok.startswith("randint"):
                k, v = tok.split(":", 1)
                self.dist[k] = v
            else:
                self.dist["samples"] = tok
        self.pool_size = int(getattr(p, "synth_pool_size", 0) or
                             os.environ.get("LBANN_NUM_PRE_GENERATED_SYNTHETIC_DATA", 0) or 0)
        self.pool: Dict[Tuple[str, int], np.ndarray] = {}
        self.base_seed = 1234567 + {"train": 0, "validate": 1, "test": 2, "tournament": 3}.get(self.role, 4)

    def total_samples(self):
        return self.n

    def _gen(self, field, index):
        dims = self._fields[field]
        rng = np.random.Generator(np.random.PCG64((self.base_seed * 1000003 + index * 7 +
                                                   {"samples": 0, "labels": 1, "responses": 2}[field])))
        if field == "labels":
            return self.one_hot(int(rng.integers(0, self.num_labels)))
        d = self.dist.get(field, "normal")
        if d == "normal":
            return rng.standard_normal(dims, dtype=np.float32)
        if d == "uniform":
            return rng.random(dims, dtype=np.float32)
        if d == "uniform_pm1":
            return rng.random(dims, dtype=np.float32) * 2 - 1
        if d == "lognormal":
            return np.exp(rng.standard_normal(dims, dtype=np.float32))
        if d.startswith("randint"):
            k = int(d.split(":")[1])
            return rng.integers(0, k, dims).astype(np.float32)
        raise ValueError(f"unknown synthetic distribution '{d}'")

    def fetch_field(self, field, index):
        if self.pool_size:
            key = (field, index % self.pool_size)
            if key not in self.pool:
                self.pool[key] = self._gen(field, key[1])
            return self.pool[key]
        return self._gen(field, index)


def _open(path):
    return gzip.open(path, "rb") if path.endswith(".gz") else open(path, "rb")


@register("mnist")
class MnistReader(DataReader):
    """IDX files (src/data_ingestion/readers/data_reader_mnist.cpp); pixels scaled to [0,1]."""

    def load(self):
        p = self.proto
        d = p.data_filedir
        with _open(os.path.join(d, p.data_filename)) as f:
            magic, n, h, w = struct.unpack(">IIII", f.read(16))
            self.images = np.frombuffer(f.read(n * h * w), dtype=np.uint8).reshape(n, 1, h, w)
        with _open(os.path.join(d, p.label_filename)) as f:
            magic, n2 = struct.unpack(">II", f.read(8))
            self.labels = np.frombuffer(f.read(n2), dtype=np.uint8)
        self.num_labels = 10
        self._fields = {"samples": (1, h, w), "labels": (10,)}

    def total_samples(self):
        return len(self.images)

    def fetch_field(self, field, index):
        if field == "samples":
            return self.images[index].astype(np.float32) / 255.0
        return self.one_hot(int(self.labels[index]))


@register("cifar10")
class Cifar10Reader(DataReader):
    """Binary batches (src/data_ingestion/readers/data_reader_cifar10.cpp)."""

    def load(self):
        d = self.proto.data_filedir
        names = ["test_batch.bin"] if self.role == "test" else [f"data_batch_{i}.bin" for i in range(1, 6)]
        recs = []
        for n in names:
            path = os.path.join(d, n)
            if os.path.exists(path):
                recs.append(np.fromfile(path, dtype=np.uint8).reshape(-1, 3073))
        data = np.concatenate(recs) if recs else np.zeros((0, 3073), dtype=np.uint8)
        self.labels = data[:, 0]
        self.images = data[:, 1:].reshape(-1, 3, 32, 32)
        self.num_labels = 10
        self._fields = {"samples": (3, 32, 32), "labels": (10,)}

    def total_samples(self):
        return len(self.images)

    def fetch_field(self, field, index):
        if field == "samples":
            return self.images[index].astype(np.float32) / 255.0
        return self.one_hot(int(self.labels[index]))


@register("imagenet", "image")
class ImageListReader(DataReader):
    """``<path> <label>`` list files decoded with OpenCV, transformed by the reader's
    transform pipeline (src/data_ingestion/readers/data_reader_image.cpp, _imagenet.cpp)."""

    def load(self):
        p = self.proto
        self.root = p.data_filedir
        self.items = []
        with open(p.data_filename if os.path.isabs(p.data_filename)
                  else os.path.join(p.data_filedir, p.data_filename)) as f:
            for line in f:
                parts = line.split()
                if parts:
                    self.items.append((parts[0], int(parts[1]) if len(parts) > 1 else 0))
        self.num_labels = self.num_labels or 1000
        self._fields = {"samples": (3, 224, 224), "labels": (self.num_labels,)}

    def total_samples(self):
        return len(self.items)

    def fetch_field(self, field, index):
        path, label = self.items[index]
        if field == "labels":
            return self.one_hot(label)
        import cv2
        img = cv2.imread(os.path.join(self.root, path), cv2.IMREAD_COLOR)
        if img is None:
            raise IOError(f"cannot read image {path}")
        return img  # HWC uint8 BGR; the transform pipeline converts to CHW float


@register("numpy")
class NumpyReader(DataReader):
    """One .npy matrix, a row per sample; optional trailing label / response column
    (src/data_ingestion/readers/data_reader_numpy.cpp)."""

    def load(self):
        p = self.proto
        self.data = np.load(os.path.join(p.data_filedir, p.data_filename), mmap_mode="r")
        width = int(np.prod(self.data.shape[1:]))
        self.has_labels = not p.disable_labels and self.num_labels > 0
        self.has_responses = not p.disable_responses and not self.has_labels and bool(p.enable_responses)
        self.feat = width - (1 if (self.has_labels or self.has_responses) else 0)
        self._fields = {"samples": (self.feat,) if self.data.ndim == 2 else tuple(self.data.shape[1:])}
        if self.has_labels:
            self._fields["labels"] = (self.num_labels,)
        if self.has_responses:
            self._fields["responses"] = (1,)

    def total_samples(self):
        return self.data.shape[0]

    def fetch_field(self, field, index):
        row = np.asarray(self.data[index], dtype=np.float32).reshape(-1)
        if field == "samples":
            return row[:self.feat].reshape(self._fields["samples"])
        if field == "labels":
            return self.one_hot(int(row[-1]))
        return row[-1:].copy()


@register("numpy_npz", "numpy_npz_conduit")
class NpzReader(DataReader):
    """.npz archive with ``data`` and optional ``labels`` / ``responses`` arrays
    (src/data_ingestion/readers/data_reader_numpy_npz.cpp)."""

    def load(self):
        p = self.proto
        z = np.load(os.path.join(p.data_filedir, p.data_filename))
        self.data = z["data"]
        scale = float(p.scaling_factor_int16) or 1.0
        self.scale = scale if self.data.dtype == np.int16 else 1.0
        self._fields = {"samples": tuple(self.data.shape[1:])}
        self.labels = z["labels"] if "labels" in z.files and not p.disable_labels else None
        self.responses = z["responses"] if "responses" in z.files and not p.disable_responses else None
        if self.labels is not None:
            self.num_labels = self.num_labels or int(self.labels.max()) + 1
            self._fields["labels"] = (self.num_labels,)
        if self.responses is not None:
            self._fields["responses"] = tuple(self.responses.shape[1:]) or (1,)

    def total_samples(self):
        return self.data.shape[0]

    def fetch_field(self, field, index):
        if field == "samples":
            return self.data[index].astype(np.float32) * self.scale
        if field == "labels":
            return self.one_hot(int(self.labels[index]))
        return np.asarray(self.responses[index], dtype=np.float32).reshape(self._fields["responses"])


@register("csv")
class CsvReader(DataReader):
    """Delimited text, one sample per row (src/data_ingestion/readers/data_reader_csv.cpp)."""

    def load(self):
        p = self.proto
        sep = p.separator or ","
        path = os.path.join(p.data_filedir, p.data_filename)
        skip = int(p.skip_rows) + (1 if p.has_header else 0)
        arr = np.loadtxt(path, delimiter=sep, skiprows=skip, dtype=np.float32, ndmin=2)
        arr = arr[:, int(p.skip_cols):]
        cols = list(range(arr.shape[1]))
        self.label_col = int(p.label_col) if (self.num_labels and not p.disable_labels) else None
        self.resp_col = int(p.response_col) if (not p.disable_responses and p.response_col) else None
        for c in (self.label_col, self.resp_col):
            if c is not None:
                cols.remove(c % arr.shape[1])
        self.arr, self.cols = arr, cols
        self._fields = {"samples": (len(cols),)}
        if self.label_col is not None:
            self._fields["labels"] = (self.num_labels,)
        if self.resp_col is not None:
            self._fields["responses"] = (1,)

    def total_samples(self):
        return self.arr.shape[0]

    def fetch_field(self, field, index):
        row = self.arr[index]
        if field == "samples":
            return row[self.cols]
        if field == "labels":
            return self.one_hot(int(row[self.label_col]))
        return row[self.resp_col:self.resp_col + 1] if self.resp_col >= 0 else row[-1:]


@register("python")
class PythonReader(DataReader):
    """A user module exposing sample / count / dims functions
    (src/data_ingestion/readers/data_reader_python.cpp:189-330); the single field is ``samples``."""

    def load(self):
        p = self.proto.python
        if p.module_dir and p.module_dir not in sys.path:
            sys.path.insert(0, p.module_dir)
        mod = importlib.import_module(p.module)
        self.sample_fn = getattr(mod, p.sample_function or "get_sample")
        self.n = int(getattr(mod, p.num_samples_function or "num_samples")())
        dims = getattr(mod, p.sample_dims_function or "sample_dims")()
        self._fields = {"samples": tuple(int(d) for d in dims)}

    def total_samples(self):
        return self.n

    def fetch_field(self, field, index):
        return np.asarray(self.sample_fn(index), dtype=np.float32).reshape(self._fields["samples"])


@register("python_dataset")
class PythonDatasetReader(DataReader):
    """A pickled ``lbann.util.data.Dataset`` (src/data_ingestion/readers/
    data_reader_python_dataset.cpp, python/lbann/util/data.py:73-160)."""

    def load(self):
        p = self.proto.python_dataset
        if p.module_dir and p.module_dir not in sys.path:
            sys.path.insert(0, p.module_dir)
        with open(p.dataset_path, "rb") as f:
            self.dataset = pickle.load(f)
        self.n = len(self.dataset)
        sd = self.dataset.get_sample_dims()
        self._fields = {}
        for k in ("sample", "label", "response", "label_reconstruction"):
            v = getattr(sd, k, None)
            if v is not None:
                name = {"sample": "samples", "label": "labels", "response": "responses"}.get(k, k)
                self._fields[name] = tuple(int(d) for d in (v if hasattr(v, "__iter__") else (v,)))
        self._cache = (None, None)

    def total_samples(self):
        return self.n

    def configure_partition(self, rank, num_io_partitions):
        if hasattr(self.dataset, "rank"):
            self.dataset.rank = rank
            self.dataset.num_io_partitions = num_io_partitions

    def fetch_field(self, field, index):
        if self._cache[0] != index:
            self._cache = (index, self.dataset[index])
        s = self._cache[1]
        attr = {"samples": "sample", "labels": "label", "responses": "response"}.get(field, field)
        return np.asarray(getattr(s, attr), dtype=np.float32).reshape(self._fields[field])


@register("hdf5", "hdf5_data_reader")
class Hdf5Reader(DataReader):
    """HDF5 files (src/data_ingestion/readers/data_reader_hdf5_legacy.cpp and the
    schema-driven data_reader_HDF5.cpp).  Needs h5py; one sample per file listed in
    ``data_filename`` or matched by ``data_file_pattern``."""

    def load(self):
        try:
            import h5py  # noqa: F401
        except ImportError as e:
            raise RuntimeError("the hdf5 reader needs the h5py package, which is not installed") from e
        import glob
        import h5py
        p = self.proto
        self.h5py = h5py
        self.files = sorted(glob.glob(os.path.join(p.data_filedir, p.data_file_pattern or "*.h5*")))
        self.kd = p.hdf5_key_data or "full"
        self.kr = p.hdf5_key_responses or "unitPar"
        with h5py.File(self.files[0], "r") as f:
            self._fields = {"samples": tuple(f[self.kd].shape)}
            if self.kr in f:
                self._fields["responses"] = (int(p.num_responses) or int(np.prod(f[self.kr].shape)),)

    def total_samples(self):
        return len(self.files)

    def fetch_field(self, field, index):
        with self.h5py.File(self.files[index], "r") as f:
            if field == "samples":
                return np.asarray(f[self.kd], dtype=np.float32)
            return np.asarray(f[self.kr], dtype=np.float32).reshape(-1)[:self._fields["responses"][0]]


@register("merge_samples")
class MergeSamplesReader(DataReader):
    """Concatenation of several readers' sample lists
    (src/data_ingestion/readers/data_reader_merge_samples.cpp)."""

    def __init__(self, readers: List[DataReader], **kw):
        super().__init__(None, **kw)
        self.readers = readers

    def load(self):
        for r in self.readers:
            r.load()
        self._fields = dict(self.readers[0].fields())
        self.offsets = np.cumsum([0] + [r.total_samples() for r in self.readers])

    def total_samples(self):
        return int(self.offsets[-1])

    def fetch_field(self, field, index):
        k = int(np.searchsorted(self.offsets, index, side="right") - 1)
        return self.readers[k].fetch_field(field, index - int(self.offsets[k]))


@register("merge_features")
class MergeFeaturesReader(DataReader):
    """Feature-wise concatenation of several readers
    (src/data_ingestion/readers/data_reader_merge_features.cpp)."""

    def __init__(self, readers: List[DataReader], **kw):
        super().__init__(None, **kw)
        self.readers = readers

    def load(self):
        for r in self.readers:
            r.load()
        width = sum(int(np.prod(r.dims("samples"))) for r in self.readers)
        self._fields = {"samples": (width,)}
        for k in ("labels", "responses"):
            if k in self.readers[-1].fields():
                self._fields[k] = self.readers[-1].dims(k)

    def total_samples(self):
        return min(r.total_samples() for r in self.readers)

    def fetch_field(self, field, index):
        if field == "samples":
            return np.concatenate([np.asarray(r.fetch_field("samples", index)).reshape(-1)
                                   for r in self.readers])
        return self.readers[-1].fetch_field(field, index)


@register("smiles")
class SmilesReader(DataReader):
    """SMILES strings tokenised with a vocabulary file into fixed-length index sequences
    (src/data_ingestion/readers/data_reader_smiles.cpp)."""

    def load(self):
        p = self.proto
        path = os.path.join(p.data_filedir, p.data_filename)
        with open(path) as f:
            rows = [ln.split()[0] for ln in f if ln.strip()]
        if p.has_header:
            rows = rows[1:]
        self.rows = rows
        vocab_path = p.metadata_filename or p.label_filename
        self.vocab = {}
        if vocab_path and os.path.exists(vocab_path):
            with open(vocab_path) as f:
                for ln in f:
                    parts = ln.split()
                    if len(parts) >= 2:
                        self.vocab[parts[0]] = int(parts[1])
        self.pad = self.vocab.get("<pad>", 0)
        self.unk = self.vocab.get("<unk>", 1)
        self.bos = self.vocab.get("<bos>", 2)
        self.eos = self.vocab.get("<eos>", 3)
        self.seq = int(os.environ.get("LBANN_SMILES_SEQUENCE_LENGTH", 0)) or \
            (max((len(r) for r in rows), default=0) + 2)
        self._fields = {"samples": (self.seq,)}

    def total_samples(self):
        return len(self.rows)

    def fetch_field(self, field, index):
        toks = [self.bos] + [self.vocab.get(c, self.unk) for c in self.rows[index]][:self.seq - 2] + [self.eos]
        toks += [self.pad] * (self.seq - len(toks))
        return np.asarray(toks, dtype=np.float32)


@register("node2vec")
class Node2VecReader(DataReader):
    """Random-walk contexts with negative samples over an edge-list graph
    (src/data_ingestion/readers/data_reader_node2vec.cpp)."""

    def load(self):
        p = self.proto.node2vec
        edges = np.loadtxt(p.graph_file, dtype=np.int64, ndmin=2)[:, :2]
        n = int(edges.max()) + 1
        self.adj = [[] for _ in range(n)]
        for a, b in edges:
            self.adj[a].append(int(b))
            self.adj[b].append(int(a))
        self.walk = int(p.walk_length) or 8
        self.neg = int(p.num_negative_samples) or 4
        self.n = int(p.epoch_size) or n
        self.num_nodes = n
        self._fields = {"samples": (self.walk + self.neg,)}

    def total_samples(self):
        return self.n

    def fetch_field(self, field, index):
        rng = np.random.RandomState(index)
        cur = index % self.num_nodes
        walk = [cur]
        for _ in range(self.walk - 1):
            nb = self.adj[cur]
            cur = nb[rng.randint(len(nb))] if nb else cur
            walk.append(cur)
        neg = rng.randint(0, self.num_nodes, self.neg).tolist()
        return np.asarray(neg + walk, dtype=np.float32)


class ArrayReader(DataReader):
    """In-memory arrays, used by ``lbann.evaluate`` and tests."""

    def __init__(self, arrays: Dict[str, np.ndarray], role="train", shuffle=False):
        super().__init__(None, role=role, shuffle=shuffle)
        self.arrays = {k: np.asarray(v, dtype=np.float32) for k, v in arrays.items()}

    def load(self):
        self._fields = {k: tuple(v.shape[1:]) or (1,) for k, v in self.arrays.items()}

    def total_samples(self):
        return len(next(iter(self.arrays.values())))

    def fetch_field(self, field, index):
        return self.arrays[field][index].reshape(self._fields[field])


@register("numpy_npz_conduit", "npz_bundle")
class SampleListReader(DataReader):
    """Bundle files selected through a sample list (``sample_list`` of the reader message).
    A bundle is an ``.npz`` archive whose arrays are called ``<sample>/<field>``; the fields
    of the first sample define the data fields.  A bounded set of bundles stays open, as in
    the reference's open-file sample lists
    (include/lbann/data_ingestion/readers/sample_list_open_files.hpp, used by
    data_reader_npz_ras_lipid.cpp / data_reader_jag_conduit.cpp)."""

    max_open_files = 16

    def load(self):
        from .sample_list import SampleList
        p = self.proto
        path = p.sample_list if os.path.isabs(p.sample_list) or not p.data_filedir \
            else os.path.join(p.data_filedir, p.sample_list)
        self.sample_list = SampleList.load(path)
        if not len(self.sample_list):
            raise ValueError(f"sample list {path} selects no samples")
        self._open_files: Dict[str, object] = {}
        first = self._bundle(0)
        name = self.sample_list.samples[0][1]
        self._fields = {}
        for key in first.files:
            s, _, f = key.partition("/")
            if s == name and f:
                self._fields[f] = tuple(first[key].shape) or (1,)
        if self.num_labels and "labels" in self._fields:
            self._fields["labels"] = (self.num_labels,)

    def _bundle(self, index):
        path = self.sample_list.path_of(index)
        z = self._open_files.get(path)
        if z is None:
            if len(self._open_files) >= self.max_open_files:
                old = next(iter(self._open_files))
                self._open_files.pop(old).close()
            z = self._open_files[path] = np.load(path)
        return z

    def total_samples(self):
        return len(self.sample_list)

    def fetch_field(self, field, index):
        a = self._bundle(index)[f"{self.sample_list.samples[index][1]}/{field}"]
        if field == "labels" and self.num_labels:
            return self.one_hot(int(np.asarray(a).reshape(-1)[0]))
        return np.asarray(a, dtype=np.float32).reshape(self._fields[field])


def build_reader(reader_pb, metadata=None) -> DataReader:
    """``metadata``: the experiment's ``DataSetMetaData`` message (key selection and
    normalisation of the JAG reader)."""
    from . import readers_science  # noqa: F401  (registers the application readers)
    name = reader_pb.name
    role = {"validation": "validate", "validate": "validate", "test": "test", "train": "train",
            "tournament": "tournament"}.get(reader_pb.role or "train", reader_pb.role)
    if name not in READER_REGISTRY:
        raise ValueError(f"unknown data reader '{name}'")
    cls = READER_REGISTRY[name]
    r = cls(reader_pb, role=role, metadata=metadata) if getattr(cls, "KINDS", None) else cls(reader_pb, role=role)
    if len(reader_pb.transforms):
        from .transforms import build_pipeline
        r.transforms = build_pipeline(reader_pb.transforms)
    return r
