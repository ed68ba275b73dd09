"""Buffered data coordinator.

Owns one reader per execution mode, deals every global mini-batch to the data-parallel
ranks, and keeps the next mini-batch in flight: a background I/O thread fetches and
collates into pinned host buffers while the current step runs, and the host-to-device copy
is issued on a dedicated CUDA stream whose completion event the compute stream waits on.
Semantics (iterations per epoch, last mini-batch size, reshuffle per epoch, per-rank sample
assignment) follow src/data_ingestion/coordinator/buffered_data_coordinator.cpp:140-420 and
data_coordinator.cpp.
"""
from __future__ import annotations

import math
import threading
import time
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .readers import DataReader

MODE_ROLE = {"training": "train", "validation": "validate", "testing": "test",
             "tournament": "tournament"}


class _ModeState:
    def __init__(self, reader: Optional[DataReader], mb: int):
        self.reader = reader
        self.mb = mb
        self.pos = 0
        self.epoch = 0
        self.order: np.ndarray = reader.indices.copy() if reader is not None else np.zeros(0, np.int64)
        self.inflight: Optional[Future] = None
        self.last_indices = np.zeros(0, np.int64)
        self.samples_fetched = 0
        self.bytes_fetched = 0
        self.fetch_seconds = 0.0


def slice_with_halo(t: torch.Tensor, dim: int, start: int, stop: int, halo: int = 0) -> torch.Tensor:
    """``t[start - halo : stop + halo]`` along ``dim``, with zeros where that leaves the tensor
    (a rank's slab of a partitioned sample together with the planes its first convolution
    reads from the neighbouring slabs)."""
    if halo <= 0:
        return t.narrow(dim, start, stop - start)
    lo, hi = start - halo, stop + halo
    a, b = max(lo, 0), min(hi, t.shape[dim])
    core = t.narrow(dim, a, b - a)
    if a == lo and b == hi:
        return core
    shape = list(t.shape)
    shape[dim] = hi - lo
    out = torch.zeros(shape, dtype=t.dtype)
    out.narrow(dim, a - lo, b - a).copy_(core)
    return out


class Batch:
    def __init__(self, tensors, global_size, indices, end_of_epoch, offset):
        self.tensors: Dict[str, torch.Tensor] = tensors
        self.global_size = global_size
        self.indices = indices
        self.end_of_epoch = end_of_epoch
        self.offset = offset
        self.event = None
        self.h2d_bytes = 0


class DataCoordinator:
    def __init__(self, readers: Dict[str, DataReader], mini_batch_size: int, *, device="cpu",
                 dp_rank: int = 0, dp_size: int = 1, seed: int = 0, io_threads: int = 2,
                 background: bool = True, fields: Optional[Sequence[str]] = None,
                 field_dtypes: Optional[Dict[str, torch.dtype]] = None):
        self.device = torch.device(device)
        self.dp_rank, self.dp_size = dp_rank, dp_size
        self.seed = seed
        self.fields = list(fields) if fields is not None else None
        self.field_dtypes = dict(field_dtypes or {})
        self.modes: Dict[str, _ModeState] = {}
        for mode, role in MODE_ROLE.items():
            self.modes[mode] = _ModeState(readers.get(role), mini_batch_size)
        self.background = background
        self.pool = ThreadPoolExecutor(max_workers=max(1, io_threads),
                                       thread_name_prefix="lbann-io") if background else None
        self.copy_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self._pinned: Dict[tuple, List[torch.Tensor]] = {}
        self._pin_idx = 0
        self.total_h2d_bytes = 0

    # ---- geometry
    def reader(self, mode) -> Optional[DataReader]:
        return self.modes[mode].reader

    def num_samples(self, mode) -> int:
        r = self.modes[mode].reader
        return r.num_samples() if r is not None else 0

    def mini_batch_size(self, mode) -> int:
        return min(self.modes[mode].mb, self.num_samples(mode)) if self.num_samples(mode) else 0

    def set_mini_batch_size(self, mode, mb: int):
        self.modes[mode].mb = int(mb)

    def iterations_per_epoch(self, mode) -> int:
        n = self.num_samples(mode)
        return int(math.ceil(n / self.modes[mode].mb)) if n else 0

    def last_mini_batch_size(self, mode) -> int:
        n, mb = self.num_samples(mode), self.modes[mode].mb
        if not n:
            return 0
        return n - (self.iterations_per_epoch(mode) - 1) * mb

    def dims(self, field: str):
        for st in self.modes.values():
            if st.reader is not None:
                return st.reader.dims(field)
        raise KeyError(field)

    def slice_points(self, which: str):
        for st in self.modes.values():
            if st.reader is not None:
                return st.reader.slice_points(which)
        raise KeyError(which)

    # ---- statistics for callbacks
    def last_indices(self, mode): return self.modes[mode].last_indices
    def samples_fetched(self, mode): return self.modes[mode].samples_fetched
    def bytes_fetched(self, mode): return self.modes[mode].bytes_fetched
    def fetch_seconds(self, mode): return self.modes[mode].fetch_seconds

    # ---- epoch handling
    def _reshuffle(self, st: _ModeState, mode: str):
        r = st.reader
        st.order = r.indices.copy()
        if r.shuffle and mode in ("training", "tournament"):
            from ..utils.random import data_order
            st.order = data_order(self.seed, st.order, st.epoch)

    def start_epoch(self, mode: str):
        st = self.modes[mode]
        if st.reader is None:
            return
        if getattr(st, "primed", False):
            # the end of the previous epoch already drew this epoch's order and started
            # fetching its first mini-batch
            st.primed = False
            st.pos = 0
            return
        if st.inflight is not None:
            st.inflight.cancel()
            try:
                st.inflight.result()
            except Exception:
                pass
            st.inflight = None
        st.pos = 0
        self._reshuffle(st, mode)

    # ---- fetching
    def _my_slice(self, global_idx: np.ndarray) -> np.ndarray:
        # deal samples round-robin to the data-parallel ranks (STAR,VC column distribution)
        return global_idx[self.dp_rank::self.dp_size]

    def _pinned_like(self, key, shape, dtype):
        bufs = self._pinned.setdefault(key, [])
        for t in bufs:
            if t.shape == shape and t.dtype == dtype and not getattr(t, "_busy", False):
                return t
        t = torch.empty(shape, dtype=dtype).pin_memory() if self.device.type == "cuda" \
            else torch.empty(shape, dtype=dtype)
        if len(bufs) >= 4:
            bufs.pop(0)
        bufs.append(t)
        return t

    def _collate(self, mode: str, pos: int) -> Batch:
        st = self.modes[mode]
        r = st.reader
        t0 = time.perf_counter()
        gidx = st.order[pos:pos + st.mb]
        mine = self._my_slice(gidx)
        fields = self.fields or list(r.fields())
        if getattr(self, "cache_collated", False):
            # Readers that cycle through a fixed pool of samples (synthetic data) keep their
            # collated, pinned mini-batches; a step then costs only the host-to-device copy.
            key = (mode, mine.tobytes())
            cache = self.__dict__.setdefault("_collated", {})
            if key in cache:
                out, nbytes = cache[key]
                st.samples_fetched += len(mine)
                b = Batch(dict(out), len(gidx), mine, pos + st.mb >= len(st.order), pos)
                b.h2d_bytes = nbytes if self.device.type == "cuda" else 0
                return b
        if getattr(r, "owner_of", None) is not None and r.world == self.dp_size and self.dp_size > 1:
            # data store: owners send the samples this rank needs (no file reads after the
            # first epoch)
            host = r.fetch_batch_global(gidx, self.dp_rank, self.dp_size, fields)
        else:
            host = r.fetch_batch(mine, fields)
        out = {}
        nbytes = 0
        for f, t in host.items():
            sl = getattr(self, "field_slices", {}).get(f)
            if isinstance(sl, list):    # a brick of the sample: one slice per partitioned dimension
                for one in sl:
                    t = slice_with_halo(t, one[0], one[1], one[2], one[3] if len(one) > 3 else 0)
            elif sl is not None:    # this rank only needs a slab of the sample (distconv)
                t = slice_with_halo(t, sl[0], sl[1], sl[2], sl[3] if len(sl) > 3 else 0)
            dt = self.field_dtypes.get(f)
            if dt is not None and t.dtype != dt:
                t = t.to(dt)
            if self.device.type == "cuda" and getattr(self, "cache_collated", False):
                out[f] = t.contiguous().pin_memory()
            elif self.device.type == "cuda":
                pin = self._pinned_like((mode, f, self._pin_idx % 3), tuple(t.shape), t.dtype)
                ev = getattr(pin, "_lb_event", None)
                if ev is not None:
                    ev.synchronize()      # the previous upload from this buffer has finished
                pin.copy_(t)
                out[f] = pin
            else:
                out[f] = t
            nbytes += t.numel() * t.element_size()
        self._pin_idx += 1
        st.samples_fetched += len(mine)
        st.bytes_fetched += nbytes
        st.fetch_seconds += time.perf_counter() - t0
        if getattr(self, "cache_collated", False):
            self.__dict__.setdefault("_collated", {})[(mode, mine.tobytes())] = (dict(out), nbytes)
        b = Batch(out, len(gidx), mine, pos + st.mb >= len(st.order), pos)
        b.h2d_bytes = nbytes if self.device.type == "cuda" else 0
        return b

    def _to_device(self, b: Batch) -> Batch:
        if self.device.type != "cuda":
            return b
        with torch.cuda.stream(self.copy_stream):
            dev = {f: t.to(self.device, non_blocking=True) for f, t in b.tensors.items()}
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        for t in b.tensors.values():
            t._lb_event = ev
        b.tensors = dev
        b.event = ev
        self.total_h2d_bytes += b.h2d_bytes
        return b

    def _submit(self, mode: str, pos: int):
        st = self.modes[mode]
        if pos >= len(st.order):
            st.inflight = None
            return
        st.inflight = self.pool.submit(self._prefetch, mode, pos) if self.pool is not None else None

    def _prefetch(self, mode: str, pos: int) -> Batch:
        """Background job: build the batch on the host AND enqueue its host-to-device copy on
        the copy stream, so that the transfer of batch k+1 runs under the compute of batch k."""
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        return self._to_device(self._collate(mode, pos))

    def next_batch(self, mode: str) -> Optional[Batch]:
        """The next mini-batch of this rank on the device (None when the epoch is over);
        the following one is already being fetched when this returns."""
        st = self.modes[mode]
        if st.reader is None or st.pos >= len(st.order):
            return None
        if st.inflight is not None:
            b = st.inflight.result()          # already on its way to the device
            st.inflight = None
        else:
            b = self._to_device(self._collate(mode, st.pos))
        st.pos += st.mb
        st.last_indices = b.indices
        if self.background:
            self._submit(mode, st.pos)
        if b.event is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(b.event)
            for t in b.tensors.values():      # allocated on the copy stream, used on this one
                t.record_stream(cur)
        if b.end_of_epoch:
            st.epoch += 1
            if self.background and self.pool is not None:
                # draw the next epoch's order now and start on its first mini-batch, so the
                # epoch boundary does not expose a host fetch and a host-to-device copy
                self._reshuffle(st, mode)
                st.pos = len(st.order)
                st.inflight = self.pool.submit(self._prefetch, mode, 0)
                st.primed = True
        return b

    def peek_batch(self, mode: str):
        """A batch of the given mode without advancing the position (gradient checks)."""
        st = self.modes[mode]
        if st.reader is None or len(st.order) == 0:
            return None
        b = self._to_device(self._collate(mode, 0))
        if b.event is not None:
            torch.cuda.current_stream(self.device).wait_event(b.event)
        return b.tensors

    # ---- checkpointing
    def state(self):
        return {m: {"pos": st.pos, "epoch": st.epoch, "order": st.order.copy(), "mb": st.mb,
                    "reader": st.reader.state() if st.reader is not None else None}
                for m, st in self.modes.items()}

    def load_state(self, state):
        for m, s in state.items():
            st = self.modes[m]
            st.pos, st.epoch, st.mb = int(s["pos"]), int(s["epoch"]), int(s["mb"])
            if st.inflight is not None:
                st.inflight.cancel()
                st.inflight = None
            st.primed = False
            st.order = np.asarray(s["order"], dtype=np.int64)
            if st.reader is not None and s.get("reader") is not None:
                st.reader.load_state(s["reader"])
            st.inflight = None

    def shutdown(self):
        if self.pool is not None:
            self.pool.shutdown(wait=False, cancel_futures=True)
