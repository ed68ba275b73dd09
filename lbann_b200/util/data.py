"""Python-side datasets (``lbann.util.data``): subclass :class:`Dataset`, pickle it with
:func:`construct_python_dataset_reader` and the ``python_dataset`` reader feeds it to
the trainer (python/lbann/util/data.py:15-439).  :class:`DataReader` is the prefetching
loader the reader drives: worker threads fetch samples ahead of the consumer.
"""
from __future__ import annotations

import os
import pickle
from abc import ABC, abstractmethod
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Union

import numpy as np


class Sample:
    """One data sample: any of ``sample``, ``label``, ``response``, ``label_reconstruction``."""

    def __init__(self, sample=None, label=None, response=None, label_reconstruction=None):
        self.sample, self.label, self.response = sample, label, response
        self.label_reconstruction = label_reconstruction


class SampleDims:
    """Dimensions of the fields a dataset provides (fields it lacks stay ``None``)."""

    def __init__(self, sample=None, label=None, response=None, label_reconstruction=None):
        self.sample, self.label, self.response = sample, label, response
        self.label_reconstruction = label_reconstruction


class Dataset(ABC):
    @abstractmethod
    def __len__(self) -> int:
        ...

    @abstractmethod
    def __getitem__(self, index: int) -> Sample:
        ...

    @abstractmethod
    def get_sample_dims(self) -> SampleDims:
        ...


class DistConvDataset(Dataset):
    """A dataset whose ``__getitem__`` returns only this rank's spatial slab: the reader
    sets ``rank`` and ``num_io_partitions`` before the first fetch."""

    _rank, _parts = 0, 1

    @property
    def rank(self) -> int:
        return self._rank

    @rank.setter
    def rank(self, r: int) -> None:
        self._rank = int(r)

    @property
    def num_io_partitions(self) -> int:
        return self._parts

    @num_io_partitions.setter
    def num_io_partitions(self, n: int) -> None:
        self._parts = int(n)


class DataReader:
    """Prefetching loader around a :class:`Dataset`."""

    def __init__(self, dataset: Dataset, num_procs: int = 2, prefetch_factor: int = 2,
                 dtype=np.float32):
        self.dataset, self.dtype = dataset, dtype
        self.dims = dataset.get_sample_dims()
        self.pool = ThreadPoolExecutor(max_workers=max(1, num_procs), thread_name_prefix="lbann-dataset")
        self.prefetch = max(1, prefetch_factor) * max(1, num_procs)
        self.pending: List = []

    def terminate(self) -> None:
        self.pool.shutdown(wait=False, cancel_futures=True)

    def queue_samples(self, inds: List[int]) -> None:
        for i in inds:
            self.pending.append(self.pool.submit(self.dataset.__getitem__, int(i)))

    def get_batch(self, batch_size: int) -> Dict[str, Union[np.ndarray, int]]:
        take, self.pending = self.pending[:batch_size], self.pending[batch_size:]
        samples = [f.result() for f in take]
        batch: Dict[str, Union[np.ndarray, int]] = {}
        for field in ("sample", "label", "response", "label_reconstruction"):
            if getattr(self.dims, field) is None:
                continue
            arr = np.stack([np.asarray(getattr(s, field), dtype=self.dtype).reshape(-1) for s in samples])
            batch[field] = arr
            batch[field + "_ptr"] = arr.ctypes.data
        return batch


def construct_python_dataset_reader(dataset: Dataset, dataset_path: Optional[str] = None,
                                    role: str = "train", prefetch_factor: int = 1,
                                    shuffle: bool = True, fraction_of_data_to_use: float = 1.0,
                                    validation_fraction: float = 0.0):
    """Pickle ``dataset`` and return the ``Reader`` message that loads it."""
    from ..proto import reader_pb2
    path = dataset_path or os.path.join(os.getcwd(), f"dataset_{role}.pkl")
    with open(path, "wb") as f:
        pickle.dump(dataset, f)
    r = reader_pb2.Reader()
    r.name = "python_dataset"
    r.role = role
    r.shuffle = shuffle
    r.fraction_of_data_to_use = fraction_of_data_to_use
    r.validation_fraction = validation_fraction
    r.python_dataset.dataset_path = path
    r.python_dataset.module_dir = os.path.dirname(os.path.abspath(
        __import__(type(dataset).__module__).__file__)) if type(dataset).__module__ != "__main__" else os.getcwd()
    r.python_dataset.prefetch_factor = prefetch_factor
    return r
