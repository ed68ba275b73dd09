"""Embedding table partitioned over the ranks of a trainer, with one-sided row access.

Row ``i`` lives on rank ``i % world`` (local row ``i // world``) in that rank's fp32 shard
of a symmetric buffer.  Forward gathers the looked-up rows straight from their owners with
peer loads; backward adds ``-learning_rate * dy`` to the owners' rows with fp32 reductions
over NVLink, which is the layer's built-in sparse SGD step applied where the row lives (no
dense gradient, no optimizer state).  Each kernel opens with a rendezvous of the group, so
rows are never read while a peer still updates them.

Replaces the reference's NVSHMEM / OpenSHMEM implementation
(src/layers/misc/dist_embedding.cu:221-360 request rows, 479-640 send gradients and apply
the sparse SGD step).  On CPU ranks (gloo) the table stays replicated and every rank
applies the gradients of all ranks, which gives the same numbers.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong as c_ll, c_void_p

import torch
import torch.distributed as dist

from ..ops import native
from . import symm

_configured = False


def _lib():
    global _configured
    lib = symm._lib()
    if not _configured:
        vpp = ctypes.POINTER(c_void_p)
        lib.lb_dist_embed_gather.restype = c_int
        lib.lb_dist_embed_gather.argtypes = [vpp, vpp, c_int, c_int, c_void_p, c_void_p, c_ll, c_int, c_ll,
                                             c_int, c_void_p, c_void_p]
        lib.lb_dist_embed_scatter.restype = c_int
        lib.lb_dist_embed_scatter.argtypes = [vpp, vpp, c_int, c_int, c_void_p, c_void_p, c_ll, c_int, c_ll,
                                              c_float, c_int, c_void_p, c_void_p]
        _configured = True
    return lib


class DistEmbeddingTable:
    """The sharded table of one layer."""

    def __init__(self, group: "symm.SymmetricGroup", weights, num: int, dim: int):
        self.group, self.weights, self.num, self.dim = group, weights, num, dim
        self.world, self.rank = group.world, group.rank
        self.rows_local = (num + self.world - 1) // self.world
        self.buf = group.alloc(self.rows_local * dim * 4)
        self.shard = self.buf.view(torch.float32, self.rows_local * dim).view(self.rows_local, dim)
        self.reload()
        # checkpoints read the live table instead of the stale replicated copy, and a
        # restart re-shards what was loaded
        weights.export_values = self.full_table
        weights.after_load = self.reload

    def reload(self):
        """(Re)build the shard from the replicated weight tensor (identical on all ranks)."""
        full = self.weights.values.detach().float().reshape(self.num, self.dim)
        mine = full[self.rank::self.world]
        self.shard.zero_()
        self.shard[:mine.shape[0]].copy_(mine)
        self.group.barrier_host()

    def full_table(self) -> torch.Tensor:
        """The whole table, read from the owners' shards (not a collective: peer rows are
        fetched by this rank's own copy kernel)."""
        out = torch.empty(self.num, self.dim, dtype=torch.float32, device=self.shard.device)
        tmp = torch.empty(self.rows_local, self.dim, dtype=torch.float32, device=self.shard.device)
        lib = symm._lib()
        row_bytes = self.dim * 4
        for r in range(self.world):
            n = len(range(r, self.num, self.world))
            if n == 0:
                continue
            if row_bytes % 16 == 0:
                rc = lib.lb_put_rows(self.buf.peer_ptr(r), row_bytes, tmp.data_ptr(), row_bytes, n,
                                     row_bytes, native.stream_ptr())
                native.check(rc, "lb_put_rows")
                out[r::self.world] = tmp[:n]
            elif r == self.rank:
                out[r::self.world] = self.shard[:n]
            else:
                raise NotImplementedError("exporting a partitioned embedding table needs "
                                          "embedding_dim to be a multiple of 4")
        return out

    def gather(self, idx: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        flat = idx.reshape(-1).contiguous()
        out = torch.empty(flat.numel(), self.dim, dtype=dtype, device=flat.device)
        rc = _lib().lb_dist_embed_gather(self.buf._c_ptrs, self.group.pad._c_ptrs, self.rank, self.world,
                                         flat.data_ptr(), out.data_ptr(), flat.numel(), self.dim, self.num,
                                         native.dtype_code(dtype), self.group.ctr_ptr,
                                         native.stream_ptr())
        native.check(rc, "lb_dist_embed_gather")
        native.count_launch()
        return out.reshape(*idx.shape, self.dim)

    def scatter_add(self, idx: torch.Tensor, dy: torch.Tensor, scale: float) -> None:
        flat = idx.reshape(-1).contiguous()
        g = dy.reshape(flat.numel(), self.dim)
        if not g.is_contiguous():
            g = g.contiguous()
        rc = _lib().lb_dist_embed_scatter(self.buf._c_ptrs, self.group.pad._c_ptrs, self.rank, self.world,
                                          flat.data_ptr(), g.data_ptr(), flat.numel(), self.dim, self.num,
                                          float(scale), native.dtype_code(g.dtype),
                                          self.group.ctr_ptr, native.stream_ptr())
        native.check(rc, "lb_dist_embed_scatter")
        native.count_launch()


class _DistEmbed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor, table: DistEmbeddingTable, idx, dtype, lr, training):
        ctx.table, ctx.idx, ctx.lr, ctx.training = table, idx, lr, training
        return table.gather(idx, dtype)

    @staticmethod
    def backward(ctx, g):
        # every rank of the group runs this backward (same graph), so the scatter kernels meet
        if ctx.training:
            ctx.table.scatter_add(ctx.idx, g, -ctx.lr)
        return torch.zeros(1, device=g.device), None, None, None, None, None


class _ReplicatedSparseSgd(torch.autograd.Function):
    """Host-side ranks: replicated table; the rows touched by ANY rank are updated on every
    rank (all-gather of indices and gradients), so the copies stay identical."""

    @staticmethod
    def forward(ctx, anchor, table, idx, lr, pg, training):
        ctx.table, ctx.idx, ctx.lr, ctx.pg, ctx.training = table, idx, lr, pg, training
        ok = (idx >= 0) & (idx < table.shape[0])
        return torch.nn.functional.embedding(idx.clamp(0, table.shape[0] - 1), table) * ok.unsqueeze(-1)

    @staticmethod
    def backward(ctx, g):
        if ctx.training:
            flat = ctx.idx.reshape(-1)
            gg = g.reshape(flat.numel(), -1).float()
            if ctx.pg is None:          # one rank: its own gradients are all there is
                all_i, all_g = [flat.cpu()], [gg.cpu()]
            else:
                world = dist.get_world_size(ctx.pg)
                sizes = [None] * world
                dist.all_gather_object(sizes, int(flat.numel()), group=ctx.pg)
                n = max(sizes)
                pad_i = torch.full((n,), -1, dtype=torch.long)
                pad_i[:flat.numel()] = flat.cpu()
                pad_g = torch.zeros(n, gg.shape[1])
                pad_g[:flat.numel()] = gg.cpu()
                all_i = [torch.empty_like(pad_i) for _ in range(world)]
                all_g = [torch.empty_like(pad_g) for _ in range(world)]
                dist.all_gather(all_i, pad_i, group=ctx.pg)
                dist.all_gather(all_g, pad_g, group=ctx.pg)
            with torch.no_grad():
                for ii, gi in zip(all_i, all_g):
                    keep = (ii >= 0) & (ii < ctx.table.shape[0])
                    ctx.table.index_add_(0, ii[keep].to(ctx.table.device),
                                         gi[keep].to(ctx.table.device, ctx.table.dtype), alpha=-ctx.lr)
        return torch.zeros(1, device=g.device), None, None, None, None, None


def dist_embedding(par, layer, idx: torch.Tensor, training: bool) -> torch.Tensor:
    """Entry point used by the ``dist_embedding`` layer when the trainer has several ranks and
    the layer runs its own sparse SGD."""
    dtype = layer.dtype or layer.model.default_dtype
    lr = float(layer.params.learning_rate)
    if getattr(layer.model, "amp_enabled", False):
        lr /= float(layer.model.amp_scale)      # the incoming gradient carries the loss scale
    anchor = getattr(layer, "_dist_anchor", None)
    if anchor is None:
        anchor = layer._dist_anchor = torch.zeros(1, device=idx.device, requires_grad=True)
    if par is not None and par.world_size > 1 and par.group.native:
        table = getattr(layer, "_dist_table", None)
        if table is None:
            table = layer._dist_table = DistEmbeddingTable(par.group, layer.w, layer.num, layer.dim)
        return _DistEmbed.apply(anchor, table, idx, dtype, lr, training)
    pg = par.comm.trainer_group if par is not None and par.world_size > 1 else None
    out = _ReplicatedSparseSgd.apply(anchor, layer.w.handle.master.detach(), idx, lr, pg, training)
    return out.to(dtype)
