"""Sample access functions for the Python data reader over ONE two-dimensional array saved
as ``data.npy`` in the working directory: row i is sample i
(python/lbann/contrib/single_tensor_data_reader.py).  Used for tests and evaluation runs:

    reader.python.module = "lbann.contrib.single_tensor_data_reader"
    reader.python.sample_function = "get_sample"
    reader.python.num_samples_function = "num_samples"
    reader.python.sample_dims_function = "sample_dims"
"""
import os

import numpy as np

_tensor = None


def _load():
    global _tensor
    if _tensor is None:
        _tensor = np.load(os.environ.get("LBANN_SINGLE_TENSOR_FILE", "data.npy"))
        if _tensor.ndim != 2:
            raise ValueError(f"data.npy must hold a matrix, found shape {_tensor.shape}")
    return _tensor


def get_sample(index):
    return _load()[index]


def num_samples():
    return _load().shape[0]


def sample_dims():
    return (_load().shape[1],)
