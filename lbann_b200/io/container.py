"""Tensor container files (native writer / reader in ``csrc/host_io.cpp``).

``save(path, tensors, meta)`` stores named tensors plus a JSON metadata blob;
``load(path)`` returns ``(tensors, meta)``.  Payloads are checksummed and written with
several threads.
"""
from __future__ import annotations

import ctypes
import json
from typing import Dict, Tuple

import numpy as np
import torch

from ..ops import native

_DT = [torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int64, torch.int32,
       torch.uint8, torch.int8, torch.int16, torch.bool]
_CODE = {d: i for i, d in enumerate(_DT)}
_configured = False


def _lib():
    global _configured
    lib = native.host_lib()
    if not _configured:
        vp, ci, cu, cull = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint64
        lib.lbh_writer_open.restype = vp
        lib.lbh_writer_open.argtypes = [ctypes.c_char_p]
        lib.lbh_writer_add.restype = ci
        lib.lbh_writer_add.argtypes = [vp, ctypes.c_char_p, cu, cu, ctypes.POINTER(cull), vp, cull]
        lib.lbh_writer_close.restype = ci
        lib.lbh_writer_close.argtypes = [vp]
        lib.lbh_reader_open.restype = vp
        lib.lbh_reader_open.argtypes = [ctypes.c_char_p]
        lib.lbh_reader_count.restype = ctypes.c_longlong
        lib.lbh_reader_count.argtypes = [vp]
        lib.lbh_reader_entry.restype = ci
        lib.lbh_reader_entry.argtypes = [vp, ctypes.c_longlong, ctypes.c_char_p, ci,
                                         ctypes.POINTER(cu), ctypes.POINTER(cu),
                                         ctypes.POINTER(cull), ctypes.POINTER(cull)]
        lib.lbh_reader_read.restype = ci
        lib.lbh_reader_read.argtypes = [vp, ctypes.c_longlong, vp]
        lib.lbh_reader_close.restype = ci
        lib.lbh_reader_close.argtypes = [vp]
        lib.lbh_gather_rows.restype = ci
        lib.lbh_gather_rows.argtypes = [vp, ctypes.POINTER(vp), ctypes.c_longlong,
                                        ctypes.c_longlong, ci]
        _configured = True
    return lib


def save(path: str, tensors: Dict[str, torch.Tensor], meta=None):
    lib = _lib()
    w = lib.lbh_writer_open(path.encode())
    if not w:
        raise IOError(f"cannot open {path} for writing")
    try:
        blob = np.frombuffer(json.dumps(meta if meta is not None else {}).encode(), dtype=np.uint8)
        items = [("__meta__", torch.from_numpy(blob.copy()))] + list(tensors.items())
        for name, t in items:
            if not isinstance(t, torch.Tensor):
                t = torch.as_tensor(np.asarray(t))
            t = t.detach().cpu().contiguous()
            dims = (ctypes.c_uint64 * 8)(*([int(d) for d in t.shape] + [0] * (8 - t.dim())))
            rc = lib.lbh_writer_add(w, name.encode(), _CODE[t.dtype], t.dim(), dims, t.data_ptr(),
                                    t.numel() * t.element_size())
            if rc != 0:
                raise IOError(f"writing '{name}' to {path} failed ({rc})")
    finally:
        if lib.lbh_writer_close(w) != 0:
            raise IOError(f"closing {path} failed")


def load(path: str) -> Tuple[Dict[str, torch.Tensor], dict]:
    lib = _lib()
    r = lib.lbh_reader_open(path.encode())
    if not r:
        raise IOError(f"cannot read container {path}")
    out, meta = {}, {}
    try:
        n = lib.lbh_reader_count(r)
        name = ctypes.create_string_buffer(4096)
        dt, nd, nb = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint64()
        dims = (ctypes.c_uint64 * 8)()
        for i in range(n):
            if lib.lbh_reader_entry(r, i, name, 4096, ctypes.byref(dt), ctypes.byref(nd), dims,
                                    ctypes.byref(nb)) != 0:
                raise IOError(f"bad entry {i} in {path}")
            shape = [int(dims[k]) for k in range(nd.value)]
            t = torch.empty(shape, dtype=_DT[dt.value])
            rc = lib.lbh_reader_read(r, i, t.data_ptr())
            if rc == -4:
                raise IOError(f"checksum mismatch for '{name.value.decode()}' in {path}")
            if rc != 0:
                raise IOError(f"reading '{name.value.decode()}' from {path} failed ({rc})")
            key = name.value.decode()
            if key == "__meta__":
                meta = json.loads(bytes(t.numpy().tobytes()).decode() or "{}")
            else:
                out[key] = t
    finally:
        lib.lbh_reader_close(r)
    return out, meta


def gather_rows(dst: torch.Tensor, rows, nthreads: int = 4):
    """dst[i] = rows[i] (numpy arrays / tensors of identical byte size), multi-threaded."""
    lib = _lib()
    n = len(rows)
    row_bytes = dst[0].numel() * dst.element_size() if n else 0
    ptrs = (ctypes.c_void_p * n)()
    keep = []
    for i, r in enumerate(rows):
        a = np.ascontiguousarray(r) if not isinstance(r, torch.Tensor) else r.contiguous().numpy()
        keep.append(a)
        ptrs[i] = a.ctypes.data
    lib.lbh_gather_rows(dst.data_ptr(), ptrs, n, row_bytes, nthreads)
    return dst
