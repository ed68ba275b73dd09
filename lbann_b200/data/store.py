"""In-memory sample cache with owner -> consumer exchange between the ranks of a trainer.

Every sample of the data set has one owner rank that keeps it in host memory: with
``preload`` the owners read their samples up front (sample ``i`` belongs to rank
``i % world``); otherwise the rank that fetches a sample first, during the first epoch,
becomes its owner.  Later epochs shuffle the samples differently, so a rank usually needs
samples that live elsewhere: for every mini-batch the owners send them to their consumers
point to point, and the file system is read exactly once per sample.  All ranks see the
same global index list, so who owns and who needs what is computed locally, without a
request round.

Takes the place of the reference's Conduit data store
(src/data_ingestion/data_store_conduit.cpp: preload 1003-1100, exchange_data_by_sample
1274-1400, owner maps 470-600).  ``spill`` / ``load_spilled`` write a rank's share of the
cache with its ownership table to node-local storage and read it back
(data_store_conduit.cpp:1600-1800, the ``--data_store_spill`` / checkpoint options): a restarted
job, or the next job on the same nodes, starts with a warm cache and reads no sample file.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist


class DataStore:
    """Wraps a reader; the coordinator calls ``fetch_batch_global`` with the whole
    mini-batch's indices and gets this rank's share back."""

    def __init__(self, reader, rank: int = 0, world: int = 1, pg=None, preload: bool = False,
                 tag: int = 0):
        self.reader = reader
        self.rank, self.world, self.pg = rank, world, pg
        self.tag = tag       # keeps the exchanges of different stores (roles) apart
        self.cache: Dict[int, Dict[str, np.ndarray]] = {}
        self.owner_of: Dict[int, int] = {}
        self.preloaded = False
        self.lock = threading.Lock()
        self.stats = {"file_reads": 0, "cache_hits": 0, "received": 0, "sent": 0}
        if preload:
            self.preload()

    # the reader's interface is passed through, so the store can stand where a reader stood
    def __getattr__(self, name):
        if name == "reader":
            raise AttributeError(name)
        return getattr(self.reader, name)

    @staticmethod
    def make_group():
        """A host-side (gloo) group for the exchanges, which run on an I/O thread and must
        not interleave with the training collectives of the main group."""
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return None
        return dist.new_group(backend="gloo")

    # ------------------------------------------------------------------ filling
    def _read(self, index: int, fields: Sequence[str]) -> Dict[str, np.ndarray]:
        self.stats["file_reads"] += 1
        return {f: np.asarray(self.reader.fetch_field(f, int(index)), dtype=np.float32) for f in fields}

    def preload(self, fields: Optional[Sequence[str]] = None):
        fields = list(fields or self.reader.fields())
        for i in self.reader.indices:
            i = int(i)
            self.owner_of[i] = i % self.world
            if self.owner_of[i] == self.rank:
                self.cache[i] = self._read(i, fields)
        self.preloaded = True

    # ------------------------------------------------------------------ per mini-batch
    def fetch_batch_global(self, gidx: Sequence[int], dp_rank: int, dp_size: int,
                           fields: Sequence[str]) -> Dict[str, torch.Tensor]:
        """``gidx``: the global mini-batch; sample k goes to data-parallel rank k % dp_size
        (the coordinator's dealing).  Returns this rank's samples, in order."""
        fields = list(fields)
        with self.lock:
            mine: List[int] = []
            send: Dict[int, List[int]] = {}
            recv: Dict[int, List[int]] = {}
            for k, i in enumerate(gidx):
                i = int(i)
                consumer = k % dp_size
                owner = self.owner_of.get(i)
                if owner is None:
                    owner = self.owner_of[i] = consumer      # first touch: the consumer reads it
                if consumer == dp_rank:
                    mine.append(i)
                    if owner != dp_rank:
                        recv.setdefault(owner, []).append(i)
                elif owner == dp_rank:
                    send.setdefault(consumer, []).append(i)
            fresh = set()
            for i in mine:
                if self.owner_of[i] == dp_rank and i not in self.cache:
                    self.cache[i] = self._read(i, fields)
                    fresh.add(i)
            got = self._exchange(send, recv, fields) if (send or recv) else {}
            self.stats["cache_hits"] += sum(1 for i in mine if i not in got and i not in fresh)
            out = {}
            for f in fields:
                rows = [got[i][f] if i in got else self.cache[i][f] for i in mine]
                dims = tuple(self.reader.dims(f))
                a = np.stack(rows) if rows else np.zeros((0,) + dims, dtype=np.float32)
                tf = getattr(self, "transforms", None)
                if tf is not None and f == "samples" and len(a):
                    a = np.stack([tf(r) for r in a])
                out[f] = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).reshape(len(mine), *dims)
            return out

    def fetch_batch(self, idx, fields):
        """Single-rank use: a plain cache in front of the reader."""
        return self.fetch_batch_global(idx, 0, 1, fields)


    # ------------------------------------------------------------------ spill / restore
    def spill(self, directory: str) -> str:
        """Write this rank's cached samples and the ownership table to
        ``<directory>/data_store_rank<r>.npz``; returns the file name.  Every rank writes its
        own file (node-local storage is fine: only the owner ever reads it back)."""
        import os
        os.makedirs(directory, exist_ok=True)
        path = os.path.join(directory, f"data_store_rank{self.rank}.npz")
        with self.lock:
            arrays = {"__owner_ids": np.asarray(sorted(self.owner_of), dtype=np.int64),
                      "__owner_ranks": np.asarray([self.owner_of[i] for i in sorted(self.owner_of)], dtype=np.int64),
                      "__meta": np.asarray([self.rank, self.world, int(self.preloaded)], dtype=np.int64)}
            for i, sample in self.cache.items():
                for f, a in sample.items():
                    arrays[f"{i}/{f}"] = a
        tmp = path + ".tmp.npz"
        np.savez(tmp, **arrays)
        os.replace(tmp, path)
        return path

    def load_spilled(self, directory: str) -> int:
        """Restore what ``spill`` wrote for this rank; returns the number of samples now in
        the cache.  The file must come from a run with the same number of ranks (ownership is
        by rank)."""
        import os
        path = os.path.join(directory, f"data_store_rank{self.rank}.npz")
        if not os.path.exists(path):
            raise FileNotFoundError(f"data store: no spilled cache for rank {self.rank} in {directory}")
        with np.load(path) as z:
            rank, world, preloaded = (int(v) for v in z["__meta"])
            if rank != self.rank or world != self.world:
                raise ValueError(f"data store: {path} was written by rank {rank} of {world}, "
                                 f"this is rank {self.rank} of {self.world}")
            with self.lock:
                self.owner_of = {int(i): int(r) for i, r in zip(z["__owner_ids"], z["__owner_ranks"])}
                self.cache = {}
                for key in z.files:
                    if key.startswith("__"):
                        continue
                    i, _, f = key.partition("/")
                    self.cache.setdefault(int(i), {})[f] = np.asarray(z[key], dtype=np.float32)
                self.preloaded = bool(preloaded)
        return len(self.cache)

    # ------------------------------------------------------------------ exchange
    def _sample_len(self, fields) -> int:
        return int(sum(int(np.prod(self.reader.dims(f))) for f in fields))

    def _pack(self, ids, fields) -> torch.Tensor:
        flat = [np.concatenate([self.cache[i][f].reshape(-1) for f in fields]) for i in ids]
        return torch.from_numpy(np.ascontiguousarray(np.stack(flat), dtype=np.float32))

    def _exchange(self, send, recv, fields):
        n = self._sample_len(fields)
        ops, bufs = [], {}
        for dst in sorted(send):
            t = self._pack(send[dst], fields)
            self.stats["sent"] += len(send[dst])
            ops.append(dist.P2POp(dist.isend, t, self._global(dst), group=self.pg, tag=self.tag))
        for src in sorted(recv):
            bufs[src] = torch.empty(len(recv[src]), n, dtype=torch.float32)
            ops.append(dist.P2POp(dist.irecv, bufs[src], self._global(src), group=self.pg, tag=self.tag))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        got = {}
        for src, ids in recv.items():
            arr = bufs[src].numpy()
            for row, i in zip(arr, ids):
                sample, off = {}, 0
                for f in fields:
                    dims = tuple(self.reader.dims(f))
                    k = int(np.prod(dims))
                    sample[f] = row[off:off + k].reshape(dims)
                    off += k
                got[i] = sample
                self.stats["received"] += 1
        return got

    def _global(self, r: int) -> int:
        """Rank within the store's group -> global rank (what the p2p calls address)."""
        if self.pg is None:
            return r
        return dist.get_global_rank(self.pg, r)
