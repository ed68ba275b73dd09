"""Parallel execution context of one trainer: data parallelism over the trainer's ranks,
the 2-D grid for sharded weights / model-parallel layers, and sub-grids.

Gradient synchronisation is this library's two-shot all-reduce kernel running directly on
the gradient arena, which is allocated in symmetric (peer-mapped) memory - no staging
copies, no per-tensor collectives (the reference launches one non-blocking NCCL allreduce
per weight tensor: include/lbann/optimizers/optimizer_impl.hpp:101-143).  The arena is
reduced in buckets on a side stream as soon as backward has produced them, overlapping
with the remaining backward computation.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import numpy as np
import torch

from .symm import SymmetricBuffer, SymmetricGroup


class ParallelContext:
    def __init__(self, comm, device):
        self.comm = comm
        self.device = torch.device(device)
        self.world_size = comm.procs_per_trainer
        self.rank = comm.rank_in_trainer
        self.group = SymmetricGroup(self.device, pg=comm.trainer_group)
        # grid: rows = tensor-parallel / shard dimension, columns = data-parallel replicas
        self.tp_size = comm.grid_height if comm.grid_height > 1 else 1
        self.dp_size = self.world_size // self.tp_size
        self.tp_rank = comm.grid_row
        self.dp_rank = comm.grid_col
        self.grads_are_sharded = False
        self._buffers: Dict[int, SymmetricBuffer] = {}
        self.grad_buffer: Optional[SymmetricBuffer] = None
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.bucket_bytes = 64 << 20
        self._subgrids = False
        self.tp = None
        self.fsdp = None

    # ------------------------------------------------------------------ data distribution
    def data_rank(self, distconv=None) -> int:
        if distconv is not None:
            return distconv.sample_group_index
        return self.dp_rank

    def data_size(self, distconv=None) -> int:
        if distconv is not None:
            return distconv.num_sample_groups
        return self.dp_size

    def interleave_samples(self, parts: List[np.ndarray]) -> np.ndarray:
        """Undo the round-robin dealing of samples to ranks (for dumps)."""
        n = sum(p.shape[0] for p in parts)
        out = np.zeros((n,) + parts[0].shape[1:], dtype=parts[0].dtype)
        for r, p in enumerate(parts):
            out[r::len(parts)][:p.shape[0]] = p
        return out

    # ------------------------------------------------------------------ model hooks
    def prepare_model(self, model):
        if self.tp_size > 1:
            from .tensor_parallel import TensorParallel
            self.tp = TensorParallel(self)

    def arena_allocator(self):
        """Allocator for the parameter arenas: fp32 buffers in symmetric memory so the
        gradient all-reduce works in place on peer-mapped addresses."""
        def alloc(numel: int, dtype: torch.dtype) -> torch.Tensor:
            es = torch.empty((), dtype=dtype).element_size()
            buf = self.group.alloc(numel * es)
            t = buf.view(dtype, numel)
            self._buffers[t.data_ptr()] = buf
            return t
        return alloc

    def sync_initial_weights(self, model):
        """All ranks of a trainer start from the trainer master's values."""
        if self.world_size > 1:
            self.comm.broadcast(model.arena.master, 0, "trainer")

    # ------------------------------------------------------------------ small reductions
    def allreduce_sum_inplace(self, t: torch.Tensor):
        if self.world_size == 1:
            return
        if t.dtype == torch.float32 and t.is_contiguous() and t.numel() <= 4096 and t.is_cuda:
            self.group.allreduce_small_(t, "sum")
        else:
            self.comm.allreduce(t, "trainer", "sum")

    def allreduce_max_inplace(self, t: torch.Tensor):
        if self.world_size == 1:
            return
        if t.dtype == torch.float32 and t.is_contiguous() and t.numel() <= 4096 and t.is_cuda:
            self.group.allreduce_small_(t, "max")
        else:
            self.comm.allreduce(t, "trainer", "max")

    def bn_reduction(self, stats_group: int):
        """(in-place sum over the statistics group, number of ranks in it) for batch norm:
        0 = all ranks of the trainer, k = groups of k consecutive ranks."""
        if stats_group == 0 or stats_group >= self.world_size:
            return self.allreduce_sum_inplace, float(self.world_size)
        if stats_group <= 1:
            return None, 1.0
        key = ("bn", stats_group)
        if key not in self.__dict__.setdefault("_groups", {}):
            base = self.comm.trainer_rank * self.comm.procs_per_trainer
            mine = None
            for g0 in range(0, self.world_size, stats_group):
                ranks = [base + r for r in range(g0, min(g0 + stats_group, self.world_size))]
                g = self.comm.new_group(ranks)
                if g0 <= self.rank < g0 + stats_group:
                    mine = (g, len(ranks))
            self._groups[key] = mine
        g, n = self._groups[key]

        def reduce_fn(t):
            self.comm.allreduce(t, g, "sum")
        return reduce_fn, float(n)

    # ------------------------------------------------------------------ gradient sync
    def sync_gradients(self, model):
        """Sum the gradient arena over the data-parallel ranks (loss terms are already
        divided by the global mini-batch size, so the sum is the mean gradient)."""
        if self.world_size == 1:
            return
        arena = model.arena
        buf = self._buffers.get(arena.grad.data_ptr())
        n = arena.total
        # The ranks of a process-grid column see the same samples: replicated layers compute
        # the same gradient tp_size times (model-parallel layers pre-multiply theirs).
        scale = 1.0 / self.tp_size
        if buf is None or not self.group.native:
            g = arena.grad[:max(n, 1)]
            self.comm.allreduce(g, "trainer", "sum")
            if scale != 1.0:
                g.mul_(scale)
            return
        es = arena.grad.element_size()
        per = max(self.bucket_bytes // es, 1 << 16)
        cur = torch.cuda.current_stream(self.device)
        if not getattr(self, "_early_hooks", False):
            self._install_early_reduce(model)
        # ranges already handed to the communication stream during backward
        done = sorted(getattr(self, "_early_ranges", []))
        self._early_ranges = []
        todo, pos = [], 0
        for off, cnt in done:
            if off > pos:
                todo.append((pos, off - pos))
            pos = max(pos, off + cnt)
        if pos < n:
            todo.append((pos, n - pos))
        # reduce the rest on the communication stream, bucket by bucket, and join afterwards
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            for start, length in todo:
                for off in range(start, start + length, per):
                    cnt = min(per, start + length - off)
                    self.group.allreduce_(buf, arena.grad.dtype, cnt, scale, off * es,
                                          blocks=32 if cnt * es >= (4 << 20) else 8)
        cur.wait_stream(self.comm_stream)

    def _install_early_reduce(self, model):
        """Large fully-connected weights that only one layer uses get a callback that starts
        their gradient all-reduce on the communication stream as soon as the layer's backward
        has written the gradient, so the transfer runs under the rest of backward (the
        reference starts one non-blocking all-reduce per weight the same way,
        include/lbann/optimizers/optimizer_impl.hpp:101-143).  The first step installs the
        callbacks and reduces everything at the end."""
        import functools
        self._early_hooks = True
        self._early_ranges = []
        if os.environ.get("LBANN_DISABLE_EARLY_GRAD_REDUCE"):
            return
        for w in model.weights:
            handle = getattr(w, "handle", None)
            if (handle is None or len(getattr(w, "users", [])) != 1 or w.slot.count < (1 << 20)
                    or handle.grad is None):
                continue
            handle.on_grad_ready = functools.partial(self._early_reduce, model, w)

    def _early_reduce(self, model, w):
        arena = model.arena
        buf = self._buffers.get(arena.grad.data_ptr())
        if buf is None or not self.group.native:
            return
        es = arena.grad.element_size()
        off = (w.slot.offset + 3) // 4 * 4
        end = (w.slot.offset + w.slot.count) // 4 * 4
        if end <= off:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.comm_stream.wait_event(ev)
        with torch.cuda.stream(self.comm_stream):
            self.group.allreduce_(buf, arena.grad.dtype, end - off, 1.0 / self.tp_size, off * es, blocks=32)
        self._early_ranges.append((off, end - off))

    # ------------------------------------------------------------------ sub-graph parallelism
    def subgrids_active(self) -> bool:
        return self._subgrids

    def cross_grid_sum(self, layer, x):
        t = x.contiguous()
        self.comm.allreduce(t, getattr(self.comm, "subgrid_peer_group", "trainer"), "sum")
        return t

    def cross_grid_sum_slice(self, layer, index, x):
        t = self.cross_grid_sum(layer, x)
        k = self.comm.num_subgrids
        w = t.shape[-1] // k
        return t[..., index * w:(index + 1) * w]

    # ------------------------------------------------------------------ tensor parallel hooks
    def tp_linear(self, layer, x):
        return self.tp.linear(layer, x)

    def tp_softmax(self, x, log):
        return self.tp.softmax(x, log)

    def dist_embedding(self, layer, idx, training):
        from .dist_embedding import dist_embedding
        return dist_embedding(self, layer, idx, training)

    def gather_sharded_weights(self, w):
        return self.fsdp.gather(w) if self.fsdp is not None else w.values.detach()

    def scatter_loaded_weights(self, model, tensors):
        return tensors
