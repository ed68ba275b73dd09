"""Spatial ("distconv") parallelism: activations partitioned along depth over the ranks of
a trainer, with halo exchange for convolutions and shuffles at strategy boundaries.

What the reference gets from DiHydrogen (distconv::tensor::Tensor with overlap regions,
distconv::Convolution's halo exchange, TensorMPICUDAShuffler) through its distconv adapters
(src/layers/distconv_adapter.cpp:172-515, src/layers/data_type_distconv_adapter.cpp:421-1154,
src/layers/learning/base_convolution.cpp:1326-1445) is done here with three differentiable
primitives over symmetric memory:

  HaloExchange   local slab [N, C, Dl, H, W] -> slab with `h` halo planes on both sides.
                 One kernel copies the slab into the extended buffer, STORES the boundary
                 planes straight into the neighbours' halo planes and runs the two group
                 rendezvous that order the stores against the neighbours' consumers.
                 Backward is one kernel too: halo gradients go back to their owners and are
                 added to the boundary planes.
  to_sample_parallel / to_spatial   redistribution between "every rank holds a depth slab
                 of all samples" and "every rank holds all of some samples" (an all-to-all
                 by peer stores), used where distconv layers meet ordinary layers.
  slab slicing   of replicated inputs (no communication).

Convolutions, pooling and entrywise layers then run their ordinary local kernels on the
slab (the convolution with zero padding in depth, because the halos carry the padding).
Parallel-strategy normalisation follows src/layers/distconv_adapter.cpp:227-336:
unspecified groups are 1, channel / filter parallelism of convolutions is rejected, and
left-over ranks multiply the sample groups.
"""
from __future__ import annotations

import os

from typing import Dict, Optional, Tuple

import torch

from ..ops import native
from .symm import SymmetricBuffer, SymmetricGroup

SPATIAL, SAMPLE, REPLICATED = "spatial", "sample", "replicated"


class Strategy:
    def __init__(self, ps, world: int):
        g = lambda n: max(int(getattr(ps, n, 0) or 0), 1)  # noqa: E731
        self.sample, self.depth = g("sample_groups"), g("depth_groups")
        self.height, self.width = g("height_groups"), g("width_groups")
        self.channel, self.filter = g("channel_groups"), g("filter_groups")
        if world == 1:
            self.sample = self.depth = self.height = self.width = self.channel = self.filter = 1
        spatial = self.depth * self.height * self.width * self.channel * self.filter
        if world % spatial:
            raise ValueError(f"parallel strategy uses {spatial} ranks, trainer has {world}")
        self.sample = world // spatial            # left-over ranks become sample groups

    def is_spatial(self) -> bool:
        return self.depth * self.height * self.width > 1


class DistconvContext:
    def __init__(self, comm, device, parallel):
        self.comm = comm
        self.device = torch.device(device)
        self.parallel = parallel
        self.world = comm.procs_per_trainer
        self.rank = comm.rank_in_trainer
        self.group: SymmetricGroup = parallel.group if parallel is not None else \
            SymmetricGroup(self.device, pg=comm.trainer_group)
        self.strategies: Dict[str, Strategy] = {}
        self.depth_groups = 1
        self.num_sample_groups = 1
        self.sample_group_index = 0
        self.depth_rank = 0
        self.dist: Dict[Tuple[str, int], str] = {}
        self._enabled: Dict[str, bool] = {}
        self._bufs: Dict[tuple, SymmetricBuffer] = {}
        self.halo_bytes = 0

    # ------------------------------------------------------------------ set-up
    def prepare_model(self, model):
        self._enabled.clear()
        depth = 1
        for l in model.layers:
            if l.parallel_strategy is None:
                continue
            st = Strategy(l.parallel_strategy, self.world)
            if l.type in ("convolution", "deconvolution") and (st.channel > 1 or st.filter > 1):
                raise ValueError(f"layer '{l.name}': channel / filter parallelism is not "
                                 f"supported for convolutions")
            if st.height > 1 or st.width > 1:
                raise NotImplementedError(
                    f"layer '{l.name}': this build partitions the depth dimension only "
                    f"(height_groups / width_groups > 1 requested)")
            self.strategies[l.name] = st
            if st.is_spatial():
                if depth not in (1, st.depth):
                    raise ValueError("all distconv layers of a model must use the same depth_groups")
                depth = st.depth
        self.depth_groups = depth
        self.num_sample_groups = self.world // depth
        # ranks of one sample group are consecutive: rank = sample_group * depth + depth_rank
        self.sample_group_index = self.rank // depth
        self.depth_rank = self.rank % depth
        if depth > 1 and self.num_sample_groups > 1:
            raise NotImplementedError("mixed sample x depth partitions need one symmetric group "
                                      "per sample group; use depth_groups == ranks per trainer")
        # inputs consumed only by distconv layers are sliced on the host before upload
        tr = getattr(model, "trainer", None)
        if depth > 1 and tr is not None and tr.data_coordinator is not None:
            slicers = {}
            for l in model.layers:
                if l.type != "input":
                    continue
                kids = [model.layers_by_name[c] for c in l.child_names]
                if kids and all(self.enabled(k) for k in kids):
                    dims = tr.data_coordinator.dims(l.params.data_field or "samples")
                    if len(dims) == 4 and dims[1] % depth == 0:
                        dl = dims[1] // depth
                        slicers[l.params.data_field or "samples"] = (2, self.depth_rank * dl,
                                                                     (self.depth_rank + 1) * dl)
            tr.data_coordinator.field_slices = slicers
            self.sliced_fields = set(slicers)
        else:
            self.sliced_fields = set()

    def enabled(self, layer) -> bool:
        hit = self._enabled.get(layer.name)       # static per layer once its dims are known
        if hit is not None:
            return hit
        st = self.strategies.get(layer.name)
        val = bool(st is not None and st.is_spatial() and layer.supports_distconv
                   and self.depth_groups > 1 and self._feasible(layer))
        if getattr(layer, "in_dims", None):
            self._enabled[layer.name] = val
        return val

    def _feasible(self, layer) -> bool:
        """Can this layer still be computed on depth slabs?  Deep in a network the depth
        extent falls below what the partition needs (a 2x pooling wants an even number of
        planes per rank, a convolution at least its halo); such layers are computed
        sample-parallel instead and the tensor is redistributed in front of them."""
        dims = layer.in_dims[0] if getattr(layer, "in_dims", None) else None
        if not dims or len(dims) != 4:
            return True
        D, P = int(dims[1]), self.depth_groups
        if D % P:
            return False
        local = D // P
        if layer.type in ("convolution", "deconvolution"):
            k, s, d = layer.ksize[0], layer.stride[0], layer.dil[0]
            return local % s == 0 and local >= (k - 1) // 2 * d and local >= 1
        if layer.type == "pooling":
            return local % layer.stride[0] == 0 and local >= layer.k[0] // 2
        return local >= 1

    # ------------------------------------------------------------------ distribution bookkeeping
    def adapt_inputs(self, model, layer, xs):
        """Redistribute the inputs of ``layer`` to the layout it computes in."""
        if self.depth_groups == 1:
            return xs
        want = SPATIAL if self.enabled(layer) else SAMPLE
        out = []
        for pn, x in zip(layer.parent_names, xs):
            have = self.dist.get(pn, REPLICATED)
            if have == want or x.dim() < 1:
                out.append(x)
            elif have == REPLICATED and want == SAMPLE:
                out.append(x[self.depth_rank::self.depth_groups])
            elif have == REPLICATED and want == SPATIAL:
                dl = x.shape[2] // self.depth_groups
                out.append(x[:, :, self.depth_rank * dl:(self.depth_rank + 1) * dl])
            elif have == SPATIAL and want == SAMPLE:
                out.append(_Redistribute.apply(x, self, True, pn))
            elif have == SAMPLE and want == SPATIAL:
                out.append(_Redistribute.apply(x, self, False, pn))
            else:
                out.append(x)
        return out

    def note_outputs(self, model, layer):
        if self.depth_groups == 1:
            return
        if layer.type == "input":
            f = layer.params.data_field or "samples"
            self.dist[layer.name] = SPATIAL if f in self.sliced_fields else REPLICATED
        else:
            self.dist[layer.name] = SPATIAL if self.enabled(layer) else SAMPLE

    # ------------------------------------------------------------------ buffers
    def buffer(self, key: tuple, nbytes: int) -> SymmetricBuffer:
        """Symmetric buffer cached per use site; allocation is collective, so every rank
        must request the same keys in the same order (they execute the same graph)."""
        b = self._bufs.get(key)
        if b is None or b.nbytes < nbytes:
            b = self.group.alloc(nbytes)
            self._bufs[key] = b
        return b

    # ------------------------------------------------------------------ layer entry points
    def convolution(self, layer, x):
        from ..ops import nn
        halo = tuple((k - 1) // 2 * d for k, d in zip(layer.ksize, layer.dil))
        hd = halo[0] if layer.nd == 3 else 0
        xe = HaloExchange.apply(x, self, hd, layer.name) if hd > 0 else x
        pad = (0,) + tuple(layer.pad[1:]) if layer.nd == 3 and hd > 0 else layer.pad
        return nn.convolution(xe, layer.w.handle, None if layer.b is None else layer.b.handle,
                              layer.ksize, pad, layer.stride, layer.dil, layer.groups,
                              layer.fused_act[0], layer.fused_act[1],
                              getattr(layer, "skip_act_grad", False))

    def deconvolution(self, layer, x):
        from ..ops import nn
        if any(k != s for k, s in zip(layer.ksize, layer.stride)):
            raise NotImplementedError("distconv deconvolution needs kernel == stride (no halo)")
        return nn.deconvolution(x, layer.w.handle, None if layer.b is None else layer.b.handle,
                                layer.ksize, layer.pad, layer.stride, layer.dil, layer.out_pad,
                                layer.groups)

    def pooling(self, layer, x):
        from ..ops import nn
        if layer.k[0] != layer.stride[0] or layer.pad[0] != 0:
            hd = (layer.k[0] - 1) // 2
            if layer.k[0] % 2 == 0 or layer.stride[0] != 1:
                raise NotImplementedError("distconv pooling with overlapping windows along depth "
                                          "needs odd windows and unit stride")
            x = HaloExchange.apply(x, self, hd, layer.name, float("-inf") if layer.mode == "max" else 0.0)
            pad = (0,) + tuple(layer.pad[1:])
            return nn.pooling(x, layer.k, pad, layer.stride, layer.mode)
        act = getattr(layer, "bwd_act", (0, 0.0))
        return nn.pooling(x, layer.k, layer.pad, layer.stride, layer.mode, act[0], act[1])

    def bn_reduction(self, layer):
        return self.parallel.allreduce_sum_inplace, float(self.world)

    def sample_loss(self, layer, kind, a, b):
        """Per-sample loss of a spatially partitioned tensor: local partial sums, summed
        over the depth ranks (mean-type losses are rescaled to the global entry count)."""
        from ..ops import nn
        part = nn.sample_loss(kind, a, b.reshape(a.shape))
        if kind in ("mean_squared_error", "mean_absolute_error"):
            part = part / self.depth_groups
        return _AllReduceSum.apply(part.reshape(-1, 1), self)

    def cross_entropy(self, layer, p, labels):
        n, C = p.shape[0], p.shape[1]
        if layer.params.use_labels:
            lab = labels.reshape(n, -1).long()
            pm = p.reshape(n, C, -1).movedim(1, -1)
            ok = (lab >= 0) & (lab < C)
            picked = pm.float().gather(2, lab.clamp(0, C - 1).unsqueeze(-1)).squeeze(-1)
            part = torch.where(ok, -torch.log(picked), torch.zeros_like(picked)).sum(1, keepdim=True)
        else:
            from ..ops import nn
            part = nn.sample_loss("cross_entropy", p, labels.to(p.dtype).reshape(p.shape)).reshape(-1, 1)
        return _AllReduceSum.apply(part, self)


class _AllReduceSum(torch.autograd.Function):
    """Sum over the depth ranks; every rank then holds the full value, and only the
    depth-rank-0 copy carries the gradient weight back (the others would double count)."""

    @staticmethod
    def forward(ctx, t, dc):
        ctx.dc = dc
        out = t.float().contiguous().clone()
        dc.parallel.allreduce_sum_inplace(out.view(-1))
        return out

    @staticmethod
    def backward(ctx, g):
        # d(total)/d(partial_r) = 1 on every rank; the loss itself is counted once per
        # sample group when the objective is formed (see DistconvContext.dist == SAMPLE rule).
        return g, None


class HaloExchange(torch.autograd.Function):
    """x: logical [N, C, Dl, H, W] (channels-last memory) -> [N, C, Dl + 2h, H, W] whose outer
    planes hold the neighbours' boundary planes (``fill`` beyond the global boundary)."""

    @staticmethod
    def forward(ctx, x, dc: DistconvContext, h: int, tag: str, fill: float = 0.0):
        N, C, Dl, H, W = x.shape
        P, r = dc.depth_groups, dc.depth_rank
        plane = H * W * C * x.element_size()
        ext_bytes = N * (Dl + 2 * h) * plane
        buf = dc.buffer(("halo_fwd", tag), ext_bytes)
        xe = buf.view(x.dtype, N * (Dl + 2 * h) * H * W * C).view(N, Dl + 2 * h, H, W, C)
        x_cl = x.permute(0, 2, 3, 4, 1)
        g = dc.group
        ctx.meta = (dc, h, tag, (N, C, Dl, H, W))
        if g.native and P == g.world and r == g.rank and not os.environ.get("LBANN_DISABLE_FUSED_HALO"):
            # interior copy, boundary fill, peer stores and both rendezvous in one launch
            xs = x_cl if x_cl.is_contiguous() else x_cl.contiguous()
            if g.halo_forward(xs, buf, N, Dl, h, plane, fill):
                dc.halo_bytes += 2 * N * h * plane
                return xe.permute(0, 4, 1, 2, 3)
        xe[:, h:h + Dl].copy_(x_cl)
        if r == 0:
            xe[:, :h].fill_(fill)
        if r == P - 1:
            xe[:, h + Dl:].fill_(fill)
        src = xe  # boundary planes are read from the interior just written
        pitch = (Dl + 2 * h) * plane
        g = dc.group
        ctx.meta = (dc, h, tag, (N, C, Dl, H, W))
        if not g.native:
            # host-side ranks (gloo): same data movement with a library all-gather
            edges = torch.stack([xe[:, h:2 * h], xe[:, Dl:Dl + h]]).contiguous()
            allp = dc.comm.all_gather(edges, "trainer")
            if r > 0:
                xe[:, :h].copy_(allp[r - 1][1])
            if r < P - 1:
                xe[:, h + Dl:].copy_(allp[r + 1][0])
            return xe.permute(0, 4, 1, 2, 3).clone()
        # neighbours must be done with the previous contents of their halo planes
        g.barrier_device(2)
        if r > 0:       # my first h planes -> upper halo of the rank above
            g.put_rows(src[:, h:2 * h], buf, r - 1, (h + Dl) * plane, N, h * plane, pitch, pitch)
        if r < P - 1:   # my last h planes -> lower halo of the rank below
            g.put_rows(src[:, Dl:Dl + h], buf, r + 1, 0, N, h * plane, pitch, pitch)
        g.barrier_device(3)
        dc.halo_bytes += 2 * N * h * plane
        ctx.meta = (dc, h, tag, (N, C, Dl, H, W))
        return xe.permute(0, 4, 1, 2, 3)

    @staticmethod
    def backward(ctx, gxe):
        dc, h, tag, (N, C, Dl, H, W) = ctx.meta
        P, r = dc.depth_groups, dc.depth_rank
        g_cl = gxe.permute(0, 2, 3, 4, 1)
        if not g_cl.is_contiguous():
            g_cl = g_cl.contiguous()
        plane = H * W * C * g_cl.element_size()
        if not dc.group.native:
            edges = torch.stack([g_cl[:, :h], g_cl[:, h + Dl:]]).contiguous()
            allp = dc.comm.all_gather(edges, "trainer")
            dx = g_cl[:, h:h + Dl].clone()
            if r > 0:
                dx[:, :h] += allp[r - 1][1]
            if r < P - 1:
                dx[:, Dl - h:] += allp[r + 1][0]
            return dx.permute(0, 4, 1, 2, 3), None, None, None, None
        # receive area: [2][N][h planes] - gradients of my boundary planes computed by neighbours
        buf = dc.buffer(("halo_bwd", tag), 2 * N * h * plane)
        pitch = (Dl + 2 * h) * plane
        grp = dc.group
        if P == grp.world and r == grp.rank and not os.environ.get("LBANN_DISABLE_FUSED_HALO"):
            dx = torch.empty((N, Dl, H, W, C), dtype=g_cl.dtype, device=g_cl.device)
            if grp.halo_backward(g_cl, buf, dx, N, Dl, h, plane):
                return dx.permute(0, 4, 1, 2, 3), None, None, None, None
        if r > 0:       # gradient of the halo I received from above goes back up
            grp.put_rows(g_cl[:, :h], buf, r - 1, N * h * plane, N, h * plane, pitch, h * plane)
        if r < P - 1:
            grp.put_rows(g_cl[:, h + Dl:], buf, r + 1, 0, N, h * plane, pitch, h * plane)
        grp.barrier_device(3)
        dx = g_cl[:, h:h + Dl].clone()
        recv = buf.view(g_cl.dtype, 2 * N * h * H * W * C).view(2, N, h, H, W, C)
        if r > 0:
            dx[:, :h] += recv[0]       # written by the rank above (its lower halo gradient)
        if r < P - 1:
            dx[:, Dl - h:] += recv[1]  # written by the rank below
        grp.barrier_device(2)          # receive area may be overwritten only after this
        return dx.permute(0, 4, 1, 2, 3), None, None, None, None


class _Redistribute(torch.autograd.Function):
    """spatial -> sample (``to_sample=True``): rank r ends up with samples r, r+P, ... of the
    full depth extent; the inverse otherwise.  All-to-all by peer stores."""

    @staticmethod
    def forward(ctx, x, dc: DistconvContext, to_sample: bool, tag: str):
        ctx.meta = (dc, to_sample, tag)
        return _redistribute(x, dc, to_sample, tag + ("/s" if to_sample else "/p"))

    @staticmethod
    def backward(ctx, g):
        dc, to_sample, tag = ctx.meta
        return _redistribute(g, dc, not to_sample, tag + ("/bs" if to_sample else "/bp")), None, None, None


def _redistribute(x, dc: DistconvContext, to_sample: bool, tag: str):
    P, r = dc.depth_groups, dc.depth_rank
    x_cl = x.permute(0, 2, 3, 4, 1).contiguous()        # N, D, H, W, C
    es = x_cl.element_size()
    grp = dc.group
    if not grp.native:
        parts = dc.comm.all_gather(x_cl, "trainer")
        if to_sample:
            out = torch.cat([p[r::P] for p in parts], dim=1)
        else:
            ns, D = x_cl.shape[0], x_cl.shape[1]
            Dl = D // P
            out = torch.empty((ns * P, Dl) + tuple(x_cl.shape[2:]), dtype=x_cl.dtype, device=x_cl.device)
            for q, p in enumerate(parts):
                out[q::P] = p[:, r * Dl:(r + 1) * Dl]
        return out.permute(0, 4, 1, 2, 3)
    if to_sample:
        N, Dl, H, W, C = x_cl.shape
        ns = (N + P - 1) // P                           # samples per rank (round-robin owner)
        slab = Dl * H * W * C * es
        buf = dc.buffer(("redist", tag), ns * P * slab)
        for q in range(P):
            rows = x_cl[q::P]
            if rows.shape[0] == 0:
                continue
            # sample j of owner q, depth slab r -> [j][r] in q's buffer
            grp.put_rows(rows, buf, q, r * slab, rows.shape[0], slab, P * slab, P * slab)
        grp.barrier_device(3)
        mine = len(range(r, N, P))
        out = buf.view(x_cl.dtype, ns * P * Dl * H * W * C).view(ns, P * Dl, H, W, C)[:mine].clone()
        grp.barrier_device(2)
        return out.permute(0, 4, 1, 2, 3)
    ns, D, H, W, C = x_cl.shape
    Dl = D // P
    slab = Dl * H * W * C * es
    # every rank owns ns samples (equal counts are required for the inverse map)
    N = ns * P
    buf = dc.buffer(("redist", tag), N * slab)
    for q in range(P):
        # my sample j (global index j*P + r), depth slab q -> row (j*P + r) of q's buffer
        src = x_cl[:, q * Dl:(q + 1) * Dl]
        grp.put_rows(src, buf, q, r * slab, ns, slab, D * H * W * C * es, P * slab)
    grp.barrier_device(3)
    out = buf.view(x_cl.dtype, N * Dl * H * W * C).view(N, Dl, H, W, C).clone()
    grp.barrier_device(2)
    return out.permute(0, 4, 1, 2, 3)
