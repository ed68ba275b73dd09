"""Sub-graph parallelism: branches of a model run on disjoint GPU subsets of a trainer.

The reference tags layers with a grid (``grid_tag`` > 0), builds one process grid per tag
out of the trainer's ranks in block order (src/utils/lbann_library.cpp:310-346), runs a
tagged layer only on the ranks of its grid (src/models/model.cpp:877-905, 1625-1636) and
moves tensors between grids at the edges of the graph with ``El::copy::TranslateBetweenGrids``
(include/lbann/layers/transform/split.hpp:135-243, sum.hpp:170-279).

Here every grid, the whole trainer (tag 0) included, holds a mini-batch the same way: global
sample ``i`` lives on the ``i % size``-th rank of the grid as local sample ``i // size``.  A
tensor therefore changes grids by sending every sample from its owner on one side to its
owner on the other: ``GridTransfer`` does that as one all-to-all-v, by peer stores through
symmetric memory on GPUs (``csrc/comm_kernels.cu::scatter_rows_kernel``, one launch with
the rendezvous inside) or through a gather on CPU ranks.  It is differentiable (the
gradient travels the opposite way) and collective: every rank of the trainer calls it, also
the ranks that neither send nor receive, and ranks that hold nothing pass and receive
empty tensors.

Untagged layers inherit the tag their parents agree on, otherwise they run on the whole
trainer (src/models/model.cpp:1041-1090).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .symm import SymmetricBuffer


class SubgridContext:
    def __init__(self, comm, device, num_subgrids: int, group=None):
        P = comm.procs_per_trainer
        if num_subgrids < 1 or P % num_subgrids:
            raise ValueError(f"cannot split {P} ranks into {num_subgrids} sub-grids")
        self.comm, self.device = comm, torch.device(device)
        self.K, self.P, self.S = num_subgrids, P, P // num_subgrids
        self.rank = comm.rank_in_trainer
        self.my_grid = 1 + self.rank // self.S
        self.index_in_grid = self.rank % self.S
        self.group = group                      # SymmetricGroup of the trainer (GPUs) or None
        comm.split_subgrids(num_subgrids)       # process groups of the grids and of the peers
        self._bufs: Dict[tuple, SymmetricBuffer] = {}
        self.dangling: List[torch.Tensor] = []  # outputs of transfers that this rank does not use
        self.bytes_moved = 0

    # ------------------------------------------------------------------ layout
    def ranks(self, tag: int) -> range:
        return range(self.P) if tag == 0 else range((tag - 1) * self.S, tag * self.S)

    def member(self, tag: int) -> bool:
        return tag == 0 or tag == self.my_grid

    def owner(self, tag: int, i: int) -> int:
        r = self.ranks(tag)
        return r[i % len(r)]

    def local_count(self, tag: int, n_global: int, rank: Optional[int] = None) -> int:
        rank = self.rank if rank is None else rank
        r = self.ranks(tag)
        if rank not in r:
            return 0
        idx = rank - r[0]
        return len(range(idx, n_global, len(r)))

    def resolve_tags(self, model) -> None:
        """Untagged layers inherit from their parents (in execution order)."""
        for l in model.layers:
            tag = getattr(l, "grid_tag", -1)
            if tag is None or tag < 0:
                tags = {p.grid_tag for p in l.parents}
                tag = tags.pop() if len(tags) == 1 else 0
            if tag > self.K:
                raise ValueError(f"layer '{l.name}' is on grid {tag}, but only {self.K} sub-grids exist")
            l.grid_tag = tag

    # ------------------------------------------------------------------ transfer
    def transfer(self, x: Optional[torch.Tensor], src: int, dst: int, n_global: int, sample_shape,
                 dtype: torch.dtype, key: str) -> Optional[torch.Tensor]:
        """``x``: this rank's samples on grid ``src`` (None when it is not a member).  Returns
        this rank's samples on grid ``dst`` (None when it is not a member)."""
        if src == dst:
            return x
        if x is None:
            x = torch.zeros((0,) + tuple(sample_shape), dtype=dtype, device=self.device, requires_grad=True)
        y = _GridTransfer.apply(x, self, src, dst, int(n_global), tuple(sample_shape), key)
        if not self.member(dst):
            if y.requires_grad:
                self.dangling.append(y)      # keeps this rank in the backward exchange
            return None
        return y

    def _move(self, x: torch.Tensor, src: int, dst: int, n: int, shape, key: str) -> torch.Tensor:
        """The data movement itself (no autograd)."""
        m_src, m_dst = len(self.ranks(src)), len(self.ranks(dst))
        mine_src = self.local_count(src, n)
        mine_dst = self.local_count(dst, n)
        assert x.shape[0] == mine_src, (x.shape, mine_src, src, dst, n)
        row = 1
        for d in shape:
            row *= int(d)
        es = x.element_size()
        g = self.group
        if g is not None and g.native and (row * es) % 16 == 0:
            cap = (n + m_dst - 1) // m_dst
            buf = self._bufs.get((key, cap, row, x.dtype))
            if buf is None:
                buf = self._bufs[(key, cap, row, x.dtype)] = g.alloc(max(cap * row * es, 16))
            dst_rank = dst_row = None
            if mine_src:
                idx_src = self.rank - self.ranks(src)[0]
                gi = torch.arange(mine_src, dtype=torch.int64) * m_src + idx_src
                dst_rank = (self.ranks(dst)[0] + gi % m_dst).to(torch.int32).to(self.device)
                dst_row = (gi // m_dst).to(torch.int32).to(self.device)
            xc = x.contiguous() if mine_src else None
            if g.scatter_rows(xc, buf, dst_rank, dst_row, mine_src, row * es):
                self.bytes_moved += mine_src * row * es
                out = buf.view(x.dtype, cap * row).view(cap, *shape)[:mine_dst]
                # the buffer is reused by the next step's transfer on this edge: hand out a copy
                return out.clone()
        # CPU ranks (or rows that are not multiples of 16 bytes): gather everything, pick mine
        cap_src = (n + m_src - 1) // m_src
        pad = torch.zeros((cap_src,) + tuple(shape), dtype=x.dtype, device=x.device)
        if mine_src:
            pad[:mine_src] = x
        parts = self.comm.all_gather(pad, "trainer")
        out = torch.zeros((mine_dst,) + tuple(shape), dtype=x.dtype, device=x.device)
        if mine_dst:
            idx_dst = self.rank - self.ranks(dst)[0]
            for j in range(mine_dst):
                i = j * m_dst + idx_dst
                out[j] = parts[self.owner(src, i)][i // m_src]
        return out

    # ------------------------------------------------------------------ sums across the grids
    def cross_grid_sum(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over the ranks that hold the same samples on the different sub-grids."""
        t = x.contiguous().clone()
        self.comm.allreduce(t, self.comm.subgrid_peer_group, "sum")
        return t


class _GridTransfer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sg: SubgridContext, src, dst, n, shape, key):
        ctx.meta = (sg, src, dst, n, shape, key)
        return sg._move(x.detach(), src, dst, n, shape, key + "/f")

    @staticmethod
    def backward(ctx, g):
        sg, src, dst, n, shape, key = ctx.meta
        if g is None:
            g = torch.zeros((sg.local_count(dst, n),) + shape, device=sg.device)
        return sg._move(g.contiguous(), dst, src, n, shape, key + "/b"), None, None, None, None, None, None
