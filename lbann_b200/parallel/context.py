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


def aligned_range(offset: int, count: int, element_size: int):
    """Largest sub-range [off, end) of [offset, offset + count) whose two ends sit on 16-byte
    boundaries of the arena (the all-reduce kernel moves 16-byte vectors)."""
    v = max(16 // element_size, 1)
    off = (offset + v - 1) // v * v
    end = (offset + count) // v * v
    return off, end


def bucket_elements(bucket_bytes: int, element_size: int) -> int:
    """Elements per gradient bucket: a whole number of 16-byte vectors."""
    v = max(16 // element_size, 1)
    return max(bucket_bytes // element_size, 1 << 16) // v * v


class _CrossGridSum(torch.autograd.Function):
    """Sum over the sub-grid peers (ranks holding the same samples on the different grids);
    the gradient of a sum is the sum of the gradients, over the same peers
    (include/lbann/layers/transform/cross_grid_sum.hpp:113-148)."""

    @staticmethod
    def forward(ctx, x, sg):
        ctx.sg = sg
        return sg.cross_grid_sum(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.sg.cross_grid_sum(g), None


class Bucket:
    """A range [start, end) of the gradient arena reduced by one kernel launch."""

    def __init__(self, start: int, end: int):
        self.start, self.end = start, end
        self.slots: List[int] = []     # trainable weights that overlap the range
        self.pending = 0               # of those, how many have not reported their gradient
        self.done = False


def plan_buckets(slots, numel: int, per: int) -> List[Bucket]:
    """Buckets of ``per`` elements covering the part of the arena that holds trainable
    weights (``slots``: (offset, count) pairs).  Ranges without a trainable weight are left
    out: nothing is reduced there."""
    out = []
    for start in range(0, numel, per):
        end = min(start + per, numel)
        if any(o < end and start < o + c for o, c in slots):
            out.append(Bucket(start, end))
    return out


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
        self.subgrid = None                # SubgridContext when the trainer is split into grids
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
            from ..ops.nn import GroupSum
            return GroupSum(self.group, self.allreduce_sum_inplace), float(self.world_size)
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
    def sync_initial_weights(self, model):
        """All ranks of a trainer start from the trainer master's values; on GPUs with more
        than one rank the optimizer update is then sharded over the ranks."""
        if self.world_size > 1:
            self.comm.broadcast(model.arena.master, 0, "trainer")
        self._setup_sharded_update(model)

    def _setup_sharded_update(self, model):
        """Reduce-scatter -> update the owned blocks -> store the new values into every rank's
        master arena, instead of all-reduce -> the same update on every rank.  Needs the
        master and gradient arenas in symmetric memory (``arena_allocator``)."""
        from ..ops.optim import ArenaShard
        from ..ops.native import c_void_p
        arena = model.arena
        if (self.world_size == 1 or not self.group.native or self.tp_size > 1
                or os.environ.get("LBANN_REPLICATED_OPTIMIZER")
                or any(s.kind == "hypergradient_adam" for s in arena.slots)):
            return
        mbuf = self._buffers.get(arena.master.data_ptr())
        gbuf = self._buffers.get(arena.grad.data_ptr())
        if mbuf is None or gbuf is None:
            return
        peers = (c_void_p * self.world_size)(*mbuf.peer_ptrs)
        arena.shard = ArenaShard(self.rank, self.world_size, peers,
                                 after_step=lambda: self.group.barrier_device(3))
        if not os.environ.get("LBANN_REPLICATED_OPTIMIZER_STATE"):
            arena.compact_state()        # moments for the owned blocks only: 1 / world of the memory

    def sync_optimizer_state(self, model):
        """Collective: optimizer state sharded by ``_setup_sharded_update`` becomes whole on
        every rank (before checkpoints and model exchanges)."""
        model.arena.gather_sharded_state(lambda t: self.comm.allreduce(t, "trainer", "sum"))

    def sync_gradients(self, model):
        """Sum the gradient arena over the data-parallel ranks (loss terms are already
        divided by the global mini-batch size, so the sum is the mean gradient).  Buckets
        whose gradients were complete during backward have been reduced on the communication
        stream already (``_install_early_reduce``); the rest follows here."""
        if self.world_size == 1:
            return
        if os.environ.get("LBANN_DIAG_SKIP_GRAD_SYNC"):
            return      # timing diagnostic only: the ranks then train on different gradients
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
        if getattr(self, "_buckets", None) is None:
            self._install_early_reduce(model)
        cur = torch.cuda.current_stream(self.device)
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            for b in self._buckets:
                if not b.done:
                    self._reduce_bucket(model, b)
        cur.wait_stream(self.comm_stream)
        for b in self._buckets:            # next step
            b.done, b.pending = False, len(b.slots)
        for w in self._hooked:
            w.handle.pending_uses = max(len(w.users), 1)

    def _reduce_bucket(self, model, b):
        arena = model.arena
        buf = self._buffers[arena.grad.data_ptr()]
        es = arena.grad.element_size()
        scale = 1.0 / self.tp_size
        big = (b.end - b.start) * es >= (4 << 20)
        if arena.shard is not None:
            self.group.reduce_scatter_owned_(buf, arena.grad.dtype, b.start, b.end,
                                             arena.shard.own_elems, scale, blocks=48 if big else 8)
        else:
            self.group.allreduce_(buf, arena.grad.dtype, b.end - b.start, scale, b.start * es,
                                  blocks=32 if big else 8)
        b.done = True

    def _install_early_reduce(self, model):
        """Cuts the gradient arena into buckets and gives every trainable weight a callback:
        when the last weight of a bucket reports its gradient complete (its layer's backward
        has run), the bucket's reduction starts on the communication stream, under the rest of
        backward.  The reference starts one non-blocking all-reduce per weight the same way
        (include/lbann/optimizers/optimizer_impl.hpp:101-143); buckets keep the launches few."""
        import functools
        from ..ops.optim import OWN_CHUNKS, CHUNK
        arena = model.arena
        es = arena.grad.element_size()
        # bucket borders sit on ownership-block borders (and therefore on 16-byte borders)
        blk = OWN_CHUNKS * CHUNK
        per = max(bucket_elements(self.bucket_bytes, es) // blk, 1) * blk
        self._buckets = plan_buckets([(w.slot.offset, w.slot.count) for w in model.weights
                                      if getattr(w, "handle", None) is not None
                                      and w.handle.grad is not None], arena.master.numel(), per)
        self._hooked = []
        early = not os.environ.get("LBANN_DISABLE_EARLY_GRAD_REDUCE")
        trainable = [w for w in model.weights if getattr(w, "handle", None) is not None
                     and w.handle.grad is not None]
        for i, w in enumerate(trainable):
            mine = [b for b in self._buckets if b.start < w.slot.offset + w.slot.count
                    and w.slot.offset < b.end]
            for b in mine:
                b.slots.append(i)
            if early:
                w.handle.pending_uses = max(len(w.users), 1)
                w.handle.on_grad_ready = functools.partial(self._grad_ready, model, mine)
                # weights that a layer uses through PyTorch autograd (not through a native
                # op that writes the arena itself) report when autograd has accumulated
                w.handle.master.register_post_accumulate_grad_hook(
                    lambda _p, h=w.handle: h.mark_ready())
                self._hooked.append(w)
        for b in self._buckets:
            b.pending = len(b.slots)

    def _grad_ready(self, model, buckets):
        for b in buckets:
            b.pending -= 1
            if b.pending == 0 and not b.done and b.slots:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(self.device))
                self.comm_stream.wait_event(ev)
                with torch.cuda.stream(self.comm_stream):
                    self._reduce_bucket(model, b)

    # ------------------------------------------------------------------ sub-graph parallelism
    def subgrids_active(self) -> bool:
        return self._subgrids

    def cross_grid_sum(self, layer, x):
        if self.subgrid is not None:
            return _CrossGridSum.apply(x, self.subgrid)
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
