"""Spatial ("distconv") parallelism: activations partitioned along depth over the ranks of
a trainer, with halo exchange for convolutions and shuffles at strategy boundaries.

What the reference gets from DiHydrogen (distconv::tensor::Tensor with overlap regions,
distconv::Convolution's halo exchange, TensorMPICUDAShuffler) through its distconv adapters
(src/layers/distconv_adapter.cpp:172-515, src/layers/data_type_distconv_adapter.cpp:421-1154,
src/layers/learning/base_convolution.cpp:1326-1445) is done here with three differentiable
primitives over symmetric memory:

  fused convolution  (GPUs) the activation lives in a symmetric buffer [N, Dl + 2h, H, W, C]
                 whose inside the producing layer writes directly; the convolution kernel
                 itself stores the boundary planes into the neighbours' halo planes, computes
                 interior tiles meanwhile and waits on per-side arrival counters only before
                 the first tile that reads a halo plane (csrc/halo_sync.cuh).  The data
                 gradient is the same kernel on the extended output gradient; the filter
                 gradient reads the extended input that forward left behind.
  HaloExchange   (CPU ranks, overlapping pooling, odd channel counts) local slab
                 [N, C, Dl, H, W] -> slab with `h` halo planes on both sides as one kernel
                 beside the consumer; backward sends halo gradients back to their owners.
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
        # channel and filter groups name the SAME ranks (input channels in, output filters out)
        spatial = self.depth * self.height * self.width * max(self.channel, self.filter)
        if world % spatial:
            raise ValueError(f"parallel strategy uses {spatial} ranks, trainer has {world}")
        self.sample = world // spatial            # left-over ranks become sample groups

    def is_spatial(self) -> bool:
        return self.depth * self.height * self.width > 1

    def is_channel(self) -> bool:
        """Partition along the first sample dimension (the "channel" dimension of [N, C, ...]
        tensors: tokens of a sequence) without any spatial split."""
        return self.channel > 1 and not self.is_spatial()


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
        self.height_groups = 1                    # second and third partitioned dimensions
        self.width_groups = 1                     # (depth x height x width grid)
        self.width_rank = 0
        self.channel_groups = 1                   # partition of the channel (token) dimension of [N, C, F] tensors
        self.channel_rank = 0
        self.input_halo: Dict[str, int] = {}      # input layer -> halo planes uploaded with it
        self.num_sample_groups = 1
        self.sample_group_index = 0
        self.depth_rank = 0
        self.height_rank = 0
        self.line_pg = {}                         # tensor dim (2 depth, 3 height, 4 width) -> process group of that line
        self.dist: Dict[Tuple[str, int], str] = {}
        self._enabled: Dict[str, bool] = {}
        self._bufs: Dict[tuple, SymmetricBuffer] = {}
        self.halo_bytes = 0
        self._halo_tensors: Dict[tuple, "HaloTensor"] = {}
        self._flags: Optional[SymmetricBuffer] = None     # arrival counters of all halo tensors
        self._local_ctr: Optional[torch.Tensor] = None
        self.interior_copies = 0          # forward / backward copies into a halo tensor (0 when
                                          # the producing layer wrote there directly)

    # ------------------------------------------------------------------ set-up
    def plan(self, model_pb) -> None:
        """Depth / sample group sizes from the prototext alone (the data coordinator, which
        deals samples to the sample groups, is built before the model is)."""
        depth = height = width = channel = 1
        for l in model_pb.layer:
            if l.HasField("parallel_strategy"):
                st = Strategy(l.parallel_strategy, self.world)
                if st.is_spatial():
                    depth, height, width = max(depth, st.depth), max(height, st.height), max(width, st.width)
                elif st.is_channel() and not l.HasField("deconvolution"):
                    channel = max(channel, st.channel)
        if depth * height * width > 1 and self.world % (depth * height * width) == 0:
            self._set_grid(depth, height, 1, width)
        elif channel > 1 and self.world % channel == 0:
            self._set_grid(1, 1, channel)

    def _set_grid(self, depth: int, height: int, channel: int = 1, width: int = 1) -> None:
        """Ranks of one sample group are consecutive and form a depth x height x width grid,
        width fastest: rank = ((sample_group * depth + depth_rank) * height + height_rank) * width
        + width_rank.  A channel partition (no spatial split) uses the same consecutive ranks
        along the channel dimension."""
        spatial = depth * height * width * channel
        self.depth_groups, self.height_groups, self.channel_groups = depth, height, channel
        self.width_groups = width
        self.num_sample_groups = self.world // spatial
        self.sample_group_index = self.rank // spatial
        self.depth_rank = (self.rank % spatial) // (height * width * channel)
        self.height_rank = (self.rank // (width * channel)) % height
        self.width_rank = (self.rank // channel) % width
        self.channel_rank = self.rank % channel

    @property
    def spatial_size(self) -> int:
        """Ranks that share one sample (depth x height x width groups, or channel_groups)."""
        return self.depth_groups * self.height_groups * self.width_groups * self.channel_groups

    @property
    def grid_mode(self) -> bool:
        """More than the depth dimension is partitioned."""
        return self.height_groups * self.width_groups > 1

    @property
    def spatial_rank(self) -> int:
        return (((self.depth_rank * self.height_groups + self.height_rank) * self.width_groups
                 + self.width_rank) * self.channel_groups + self.channel_rank)

    @property
    def fused(self) -> bool:
        """The peer-memory kernels (halo exchange inside the convolutions, all-to-all
        redistribution, small all-reduce) serve the depth-only partition; a depth x height
        grid exchanges its halos with library collectives over the grid's lines."""
        return self.group.native and not self.grid_mode and self.channel_groups == 1

    def prepare_model(self, model):
        self._enabled.clear()
        depth = height = width = channel = 1
        for l in model.layers:
            if l.parallel_strategy is None:
                continue
            st = Strategy(l.parallel_strategy, self.world)
            if l.type == "deconvolution" and (st.channel > 1 or st.filter > 1):
                raise ValueError(f"layer '{l.name}': channel / filter parallelism is not "
                                 f"supported for transposed convolutions")
            if l.type == "convolution" and (st.channel > 1 or st.filter > 1):
                if st.is_spatial():
                    raise ValueError(f"layer '{l.name}': channel / filter parallelism cannot be "
                                     f"combined with a spatial partition")
                if st.filter not in (1, st.channel) or st.channel == 1:
                    raise ValueError(f"layer '{l.name}': a channel / filter partition needs "
                                     f"channel_groups == filter_groups")
            self.strategies[l.name] = st
            if st.is_spatial():
                if (depth, height, width) not in ((1, 1, 1), (st.depth, st.height, st.width)):
                    raise ValueError("all distconv layers of a model must use the same "
                                     "depth_groups, height_groups and width_groups")
                depth, height, width = st.depth, st.height, st.width
            elif st.is_channel() and l.type != "deconvolution":
                if channel not in (1, st.channel):
                    raise ValueError("all channel-partitioned layers of a model must use the same channel_groups")
                channel = st.channel
        if channel > 1 and depth * height * width > 1:
            raise ValueError("channel_groups cannot be combined with spatial partitions in one model")
        self._set_grid(depth, height, channel, width)
        self.depth_pg = "trainer"
        self.line_pg = {2: "trainer", 3: "trainer", 4: "trainer"}
        if channel > 1:
            # ranks that share a sample: consecutive groups of `channel` ranks
            if self.num_sample_groups > 1:
                base = self.comm.trainer_rank * self.world
                for sgi in range(self.num_sample_groups):
                    pg = self.comm.new_group([base + sgi * channel + i for i in range(channel)])
                    if sgi == self.sample_group_index:
                        self.depth_pg = pg
        elif height * width > 1:
            self._build_grid_groups(depth, height, width)
        elif depth > 1 and self.num_sample_groups > 1:
            # sample x depth partition (left-over ranks multiply the sample groups,
            # src/layers/distconv_adapter.cpp:227-336): the mini-batch is dealt to the sample
            # groups, every group splits its samples along depth over its own ranks and has
            # its own symmetric memory; gradients and batch-norm statistics still span the
            # whole trainer
            base = self.comm.trainer_rank * self.world
            for sgi in range(self.num_sample_groups):
                ranks = [base + sgi * depth + i for i in range(depth)]
                pg = self.comm.new_group(ranks)
                if sgi == self.sample_group_index:
                    self.depth_pg = pg
            self.group = SymmetricGroup(self.device, pg=self.depth_pg)
        # inputs consumed only by distconv layers are sliced on the host before upload
        tr = getattr(model, "trainer", None)
        if height * width > 1 and tr is not None and tr.data_coordinator is not None:
            slicers = {}
            for l in model.layers:
                if l.type != "input":
                    continue
                kids = [model.layers_by_name[c] for c in l.child_names]
                f = l.params.data_field or "samples"
                dims = tr.data_coordinator.dims(f)
                # [C, D, H, W] volumes and [D, H, W] per-voxel labels: depth is third from last
                if (kids and all(self.enabled(k) for k in kids) and len(dims) in (3, 4)
                        and dims[-3] % depth == 0 and dims[-2] % height == 0 and dims[-1] % width == 0):
                    dl, hl, wl = dims[-3] // depth, dims[-2] // height, dims[-1] // width
                    ax = len(dims) - 2            # depth axis of the mini-batch tensor
                    slicers[f] = [(ax, self.depth_rank * dl, (self.depth_rank + 1) * dl, 0),
                                  (ax + 1, self.height_rank * hl, (self.height_rank + 1) * hl, 0)]
                    if width > 1:
                        slicers[f].append((ax + 2, self.width_rank * wl, (self.width_rank + 1) * wl, 0))
                    self.input_halo[l.name] = 0
            tr.data_coordinator.field_slices = slicers
            self.sliced_fields = set(slicers)
        elif depth > 1 and tr is not None and tr.data_coordinator is not None:
            slicers = {}
            for l in model.layers:
                if l.type != "input":
                    continue
                kids = [model.layers_by_name[c] for c in l.child_names]
                if kids and all(self.enabled(k) for k in kids):
                    dims = tr.data_coordinator.dims(l.params.data_field or "samples")
                    # [C, D, H, W] volumes and [D, H, W] per-voxel labels: depth is third from last
                    if len(dims) in (3, 4) and dims[-3] % depth == 0:
                        dl = dims[-3] // depth
                        # an input read by one convolution only is uploaded WITH its halo
                        # planes (zeros beyond the volume): the first layer then needs no
                        # exchange at all
                        h = self._input_halo(kids) if (self.fused and len(dims) == 4) else 0
                        slicers[l.params.data_field or "samples"] = (len(dims) - 2, self.depth_rank * dl,
                                                                     (self.depth_rank + 1) * dl, h)
                        self.input_halo[l.name] = h
            tr.data_coordinator.field_slices = slicers
            self.sliced_fields = set(slicers)
        else:
            self.sliced_fields = set()

    def _build_grid_groups(self, depth: int, height: int, width: int = 1) -> None:
        """Process groups of a depth x height x width grid: the ranks of this sample group (sums
        of partial losses, redistribution) and the lines through this rank (halo exchange along
        depth, height and width; src/layers/distconv_adapter.cpp:227-336 sets up the same
        locale shapes).  Every rank creates every group, in the same order."""
        spatial = depth * height * width
        base = self.comm.trainer_rank * self.world
        extent = (depth, height, width)
        me = (self.depth_rank, self.height_rank, self.width_rank)

        def rank_of(c):
            return (c[0] * height + c[1]) * width + c[2]

        for sgi in range(self.num_sample_groups):
            first = base + sgi * spatial
            mine = sgi == self.sample_group_index
            if self.num_sample_groups > 1:
                pg = self.comm.new_group([first + i for i in range(spatial)])
                if mine:
                    self.depth_pg = pg
            for axis in range(3):                     # lines along `axis`: the other two coordinates fixed
                if extent[axis] == 1:
                    continue
                o1, o2 = [a for a in range(3) if a != axis]
                for c1 in range(extent[o1]):
                    for c2 in range(extent[o2]):
                        coords = []
                        for i in range(extent[axis]):
                            c = [0, 0, 0]
                            c[axis], c[o1], c[o2] = i, c1, c2
                            coords.append(first + rank_of(c))
                        pg = self.comm.new_group(coords)
                        if mine and me[o1] == c1 and me[o2] == c2:
                            self.line_pg[2 + axis] = pg

    def _input_halo(self, kids) -> int:
        """Halo planes to upload with an input: what its only consumer, a stride-1 3-D
        convolution with "same" padding along depth, reads from the neighbouring slabs
        (layers are not set up yet at this point: the numbers come from the prototext)."""
        if len(kids) != 1 or kids[0].type != "convolution":
            return 0
        from ..exec.layer_base import broadcast_list
        p = kids[0].params
        nd = int(p.num_dims) or 3
        if nd != 3:
            return 0
        k = broadcast_list(p.kernel_size, nd, 1)[0]
        s = broadcast_list(p.stride, nd, 1)[0]
        pad = broadcast_list(p.padding, nd, 0)[0]
        d = broadcast_list(p.dilation, nd, 1)[0]
        h = (k - 1) // 2 * d
        return h if (s == 1 and pad == h) else 0

    def enabled(self, layer) -> bool:
        hit = self._enabled.get(layer.name)       # static per layer once its dims are known
        if hit is not None:
            return hit
        st = self.strategies.get(layer.name)
        if self.channel_groups > 1:
            val = bool(st is not None and st.is_channel() and getattr(layer, "supports_channel_parallel", False)
                       and self._feasible_channel(layer))
        else:
            val = bool(st is not None and st.is_spatial() and layer.supports_distconv
                       and self.spatial_size > 1 and self._feasible(layer))
        if getattr(layer, "in_dims", None):
            self._enabled[layer.name] = val
        return val

    def _feasible_channel(self, layer) -> bool:
        """Channel (token) partition: every input is [C, ...] with at least two dimensions and C
        divisible by the number of ranks."""
        dims = getattr(layer, "in_dims", None)
        if not dims:
            return True
        if layer.type == "convolution" and (layer.groups != 1 or layer.cout % self.channel_groups):
            return False
        return all(len(d) >= 2 and int(d[0]) % self.channel_groups == 0 for d in dims)

    def _feasible(self, layer) -> bool:
        """Can this layer still be computed on depth slabs?  Deep in a network the depth
        extent falls below what the partition needs (a 2x pooling wants an even number of
        planes per rank, a convolution at least its halo); such layers are computed
        sample-parallel instead and the tensor is redistributed in front of them."""
        dims = layer.in_dims[0] if getattr(layer, "in_dims", None) else None
        if not dims or len(dims) != 4:
            return True
        for axis, P in ((0, self.depth_groups), (1, self.height_groups), (2, self.width_groups)):
            if P == 1:
                continue
            D = int(dims[1 + axis])
            if D % P:
                return False
            local = D // P
            if layer.type in ("convolution", "deconvolution"):
                k, s, d = layer.ksize[axis], layer.stride[axis], layer.dil[axis]
                if not (local % s == 0 and local >= (k - 1) // 2 * d and local >= 1):
                    return False
            elif layer.type == "pooling":
                if not (local % layer.stride[axis] == 0 and local >= layer.k[axis] // 2):
                    return False
            elif local < 1:
                return False
        return True

    # ------------------------------------------------------------------ distribution bookkeeping
    def adapt_inputs(self, model, layer, xs):
        """Redistribute the inputs of ``layer`` to the layout it computes in."""
        if self.spatial_size == 1:
            return xs
        want = SPATIAL if self.enabled(layer) else SAMPLE
        out = []
        for pn, x in zip(layer.parent_names, xs):
            have = self.dist.get(pn, REPLICATED)
            if have == want or x.dim() < 1:
                out.append(x)
            elif have == REPLICATED and want == SAMPLE:
                out.append(x[self.spatial_rank::self.spatial_size])
            elif have == REPLICATED and want == SPATIAL and self.channel_groups > 1:
                cl = x.shape[1] // self.channel_groups
                out.append(x.narrow(1, self.channel_rank * cl, cl))
            elif have == REPLICATED and want == SPATIAL:
                # depth is the third dimension from the last ([N, C, D, H, W] and [N, D, H, W])
                ax = x.dim() - 3
                dl = x.shape[ax] // self.depth_groups
                x = x.narrow(ax, self.depth_rank * dl, dl)
                if self.height_groups > 1:
                    hl = x.shape[ax + 1] // self.height_groups
                    x = x.narrow(ax + 1, self.height_rank * hl, hl)
                if self.width_groups > 1:
                    wl = x.shape[ax + 2] // self.width_groups
                    x = x.narrow(ax + 2, self.width_rank * wl, wl)
                out.append(x)
            elif have == SPATIAL and want == SAMPLE:
                out.append(_Redistribute.apply(x, self, True, pn))
            elif have == SAMPLE and want == SPATIAL:
                out.append(_Redistribute.apply(x, self, False, pn))
            else:
                out.append(x)
        return out

    def note_outputs(self, model, layer):
        if self.spatial_size == 1:
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
    def allreduce_depth_(self, t: torch.Tensor):
        """In-place sum over the ranks that share this rank's samples (its depth group)."""
        if self.spatial_size == 1:
            return
        if self.fused and t.dtype == torch.float32 and t.is_contiguous() and t.numel() <= 4096:
            self.group.allreduce_small_(t, "sum")
        else:
            self.comm.allreduce(t, self.depth_pg, "sum")

    def step_barrier(self):
        """Stream-ordered rendezvous of the trainer's ranks (needed between two steps that
        have no other collective between them, see csrc/halo_sync.cuh)."""
        if self.depth_groups > 1 and self.fused:
            self.group.barrier_device(3)

    def halo_tensor(self, key: tuple, N, Dl, h, H, W, C, dtype) -> "HaloTensor":
        """The symmetric tensor with halo planes of one use site (collective on first use:
        every rank runs the same graph and asks in the same order)."""
        full_key = key + (N, Dl, h, H, W, C, dtype)
        t = self._halo_tensors.get(full_key)
        if t is None:
            if self._flags is None:
                self._flags = self.group.alloc(4096 * 4)
                self._flags.local.zero_()
                self._local_ctr = torch.zeros(4096, dtype=torch.int32, device=self.device)
                self.group.barrier_host()
            t = HaloTensor(self, len(self._halo_tensors), full_key, N, Dl, h, H, W, C, dtype)
            self._halo_tensors[full_key] = t
        return t

    def _fused_halo_ok(self, layer, x, hd: int) -> bool:
        if not (self.fused and hd > 0 and x.is_cuda and layer.nd == 3 and layer.groups == 1):
            return False
        if os.environ.get("LBANN_DISTCONV_HALO_EXCHANGE", "").upper() == "SEPARATE":
            return False
        Kout, Cin = layer.w.handle.master.shape[0], layer.w.handle.master.shape[1]
        return (Kout % 8 == 0 and Cin % 8 == 0 and tuple(layer.stride) == (1, 1, 1)
                and layer.pad[0] == hd and x.shape[2] > 2 * hd - 1 and x.shape[2] >= hd
                and x.dtype in (torch.float16, torch.bfloat16)
                and (x.shape[3] * x.shape[4] * Cin * 2) % 16 == 0
                and self.depth_groups == self.group.world)

    def convolution(self, layer, x, fuse_pool=None, pool_layer=None):
        """``fuse_pool`` / ``pool_layer``: the 2^3 max pooling behind this convolution may run
        inside its kernel (ops/nn.py, PoolFusion); only the path without an exchange takes it."""
        from ..ops import nn
        if self.channel_groups > 1:
            return self._channel_convolution(layer, x)
        halo = tuple((k - 1) // 2 * d for k, d in zip(layer.ksize, layer.dil))
        if self.grid_mode:
            return self._grid_convolution(layer, x, halo)
        hd = halo[0] if layer.nd == 3 else 0
        parent = layer.parent_names[0] if layer.parent_names else None
        pre = self.input_halo.get(parent, 0)
        if hd > 0 and pre == hd:
            # the input was uploaded with its halo planes: an ordinary convolution, no exchange
            pad = (0,) + tuple(layer.pad[1:])
            if fuse_pool is not None and pool_layer is not None:
                fuse_pool.out_alloc = self._pool_allocs(pool_layer, x)[0]
            return nn.convolution(x, layer.w.handle, None if layer.b is None else layer.b.handle,
                                  layer.ksize, pad, layer.stride, layer.dil, layer.groups,
                                  layer.fused_act[0], layer.fused_act[1],
                                  getattr(layer, "skip_act_grad", False), fuse_pool)
        if self._fused_halo_ok(layer, x, hd):
            return _DistConv.apply(x, layer.w.handle.master,
                                   None if layer.b is None else layer.b.handle.master, self, layer, hd)
        xe = HaloExchange.apply(x, self, hd, layer.name) if hd > 0 else x
        pad = (0,) + tuple(layer.pad[1:]) if layer.nd == 3 and hd > 0 else layer.pad
        return nn.convolution(xe, layer.w.handle, None if layer.b is None else layer.b.handle,
                              layer.ksize, pad, layer.stride, layer.dil, layer.groups,
                              layer.fused_act[0], layer.fused_act[1],
                              getattr(layer, "skip_act_grad", False))

    def _channel_convolution(self, layer, x):
        """Channel / filter partition (src/layers/learning/base_convolution.cpp with
        channel_groups == filter_groups): the input arrives split along its channels, every rank
        gathers it, applies ITS block of filters and leaves the output split along the filters.
        The kernel stays whole on every rank; a rank's gradient is non-zero in its filter rows
        only and the sum over the ranks puts the rows together."""
        import torch.nn.functional as F
        from ..ops.gemm import _ACT_FN
        P, r = self.channel_groups, self.channel_rank
        xg = _GatherChannels.apply(x, self)
        kl = layer.cout // P
        w = layer.w.handle.master[r * kl:(r + 1) * kl]
        b = None if layer.b is None else layer.b.handle.master[r * kl:(r + 1) * kl]
        if w.dtype != xg.dtype:
            w, b = w.to(xg.dtype), (None if b is None else b.to(xg.dtype))
        fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[layer.nd]
        y = fn(xg, w, b, tuple(layer.stride), tuple(layer.pad), tuple(layer.dil), 1)
        return _ACT_FN[layer.fused_act[0]](y, layer.fused_act[1])

    def _grid_convolution(self, layer, x, halo):
        """Convolution on a depth x height (x width) grid: the halo planes along depth are
        exchanged first, then the halo rows along height of the depth-extended tensor, then the
        halo columns along width, which brings the edge and corner regions from the diagonal
        neighbours in two or three hops
        (src/layers/learning/base_convolution.cpp:1355-1445 exchanges per dimension likewise)."""
        from ..ops import nn
        if layer.nd != 3:
            raise NotImplementedError("a grid partition needs 3-D convolutions")
        parts = (self.depth_groups, self.height_groups, self.width_groups)
        pad = list(layer.pad)
        xe = x
        for axis in (0, 1, 2):
            if parts[axis] == 1:
                continue
            if layer.pad[axis] != halo[axis]:
                raise NotImplementedError(
                    f"layer '{layer.name}': a partitioned dimension needs padding (k - 1) / 2 * dilation")
            if halo[axis] > 0:
                xe = LineHaloExchange.apply(xe, self, halo[axis], 2 + axis, 0.0)
            pad[axis] = 0
        return nn.convolution(xe, layer.w.handle, None if layer.b is None else layer.b.handle,
                              layer.ksize, tuple(pad), layer.stride, layer.dil, layer.groups,
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
        if self.channel_groups > 1:            # every channel is pooled by itself
            act = getattr(layer, "bwd_act", (0, 0.0))
            return nn.pooling(x, layer.k, layer.pad, layer.stride, layer.mode, act[0], act[1])
        if self.grid_mode:
            parts = (self.depth_groups, self.height_groups, self.width_groups)
            if any(layer.k[a] != layer.stride[a] or layer.pad[a] != 0 for a in range(3) if parts[a] > 1):
                raise NotImplementedError("pooling on a grid partition needs windows that "
                                          "do not overlap (kernel == stride, no padding)")
            act = getattr(layer, "bwd_act", (0, 0.0))
            return nn.pooling(x, layer.k, layer.pad, layer.stride, layer.mode, act[0], act[1])
        if layer.k[0] != layer.stride[0] or layer.pad[0] != 0:
            hd = (layer.k[0] - 1) // 2
            if layer.k[0] % 2 == 0 or layer.stride[0] != 1:
                raise NotImplementedError("distconv pooling with overlapping windows along depth "
                                          "needs odd windows and unit stride")
            x = HaloExchange.apply(x, self, hd, layer.name, float("-inf") if layer.mode == "max" else 0.0)
            pad = (0,) + tuple(layer.pad[1:])
            return nn.pooling(x, layer.k, pad, layer.stride, layer.mode)
        act = getattr(layer, "bwd_act", (0, 0.0))
        out_alloc, dx_alloc = self._pool_allocs(layer, x)
        return nn.pooling(x, layer.k, layer.pad, layer.stride, layer.mode, act[0], act[1],
                          out_alloc, dx_alloc)

    def _pool_allocs(self, layer, x):
        """Where a pooling layer's output and input gradient go: straight into the next
        convolution's tensor with halo planes and into the producing convolution's."""
        out_alloc = dx_alloc = None
        if self.fused and x.is_cuda:
            # write the output straight into the next convolution's tensor with halo planes,
            # and the input gradient into the producing convolution's (no interior copies)
            model = getattr(layer, "model", None)
            kids = [model.layers_by_name[c] for c in layer.child_names] if model is not None else []
            if len(kids) == 1 and kids[0].type == "convolution" and self.enabled(kids[0]):
                k = kids[0]
                hk = (k.ksize[0] - 1) // 2 * k.dil[0] if k.nd == 3 else 0

                def out_alloc(shape, dtype, k=k, hk=hk):
                    N, Do, Ho, Wo, C = shape
                    probe = torch.empty((N, C, Do, Ho, Wo), dtype=dtype, device="meta")
                    if not self._fused_halo_ok(k, _Shape(probe, self.device), hk):
                        return None
                    return self.halo_tensor(("x", k.name), N, Do, hk, Ho, Wo, C, dtype).interior
            par = model.layers_by_name.get(layer.parent_names[0]) if model is not None else None
            while par is not None and getattr(par, "fused_into_parent", False) and par.parent_names:
                par = model.layers_by_name.get(par.parent_names[0])   # an activation folded into its producer
            if (par is not None and par.type == "convolution" and self.enabled(par)
                    and getattr(par, "skip_act_grad", False)):
                hp = (par.ksize[0] - 1) // 2 * par.dil[0] if par.nd == 3 else 0

                def dx_alloc(shape, dtype, par=par, hp=hp):
                    N, D, H, W, C = shape
                    if not getattr(par, "_fused_halo", False) or not getattr(par, "_needs_dx", False):
                        return None
                    return self.halo_tensor(("dy", par.name), N, D, hp, H, W, C, dtype).interior
        return out_alloc, dx_alloc

    def gather_channels(self, x):
        """The whole channel (token) extent of a channel-partitioned tensor on every rank of the
        group: the second operand of a matrix product whose first operand stays partitioned
        (scores = Q_local K^T need all keys; src/layers/math/matmul.cpp:82-130 partitions the
        same way)."""
        return _GatherChannels.apply(x, self)

    def bn_reduction(self, layer):
        from ..ops.nn import GroupSum
        # statistics span all samples and all slabs: the whole trainer, not only the depth group
        return GroupSum(self.parallel.group, self.parallel.allreduce_sum_inplace), float(self.world)

    def sample_loss(self, layer, kind, a, b):
        """Per-sample loss of a spatially partitioned tensor: local partial sums, summed
        over the depth ranks (mean-type losses are rescaled to the global entry count)."""
        from ..ops import nn
        part = nn.sample_loss(kind, a, b.reshape(a.shape))
        if kind in ("mean_squared_error", "mean_absolute_error"):
            part = part / self.spatial_size
        return _AllReduceSum.apply(part.reshape(-1, 1), self)

    def cross_entropy(self, layer, p, labels):
        n, C = p.shape[0], p.shape[1]
        if layer.params.use_labels:
            from ..exec.layer_base import rows2d
            lab = rows2d(labels).long()
            pm = p.reshape(n, C, -1).movedim(1, -1)
            ok = (lab >= 0) & (lab < C)
            picked = pm.float().gather(2, lab.clamp(0, C - 1).unsqueeze(-1)).squeeze(-1)
            part = torch.where(ok, -torch.log(picked), torch.zeros_like(picked)).sum(1, keepdim=True)
        else:
            from ..ops import nn
            part = nn.sample_loss("cross_entropy", p, labels.to(p.dtype).reshape(p.shape)).reshape(-1, 1)
        return _AllReduceSum.apply(part, self)


class _Shape:
    """Stand-in for a tensor of which only shape / dtype / device matter."""

    def __init__(self, meta: torch.Tensor, device):
        self.shape, self.dtype = meta.shape, meta.dtype
        self.is_cuda = torch.device(device).type == "cuda"


class HaloTensor:
    """A rank's [N, Dl + 2h, H, W, C] activation in symmetric memory plus what the fused
    kernels need to exchange its halo planes: the neighbours' peer-mapped copies and the
    arrival counters (two 32-bit words per tensor in a symmetric flag buffer; the launch
    counters are local).  Planes beyond the global boundary stay zero: nobody writes them."""

    def __init__(self, dc: "DistconvContext", slot: int, key, N, Dl, h, H, W, C, dtype):
        from ..ops.conv import HaloSyncArgs
        if slot >= 2048:
            raise RuntimeError("too many tensors with halo planes")
        es = torch.empty((), dtype=dtype).element_size()
        n = N * (Dl + 2 * h) * H * W * C
        self.buf = dc.buffer(("halo",) + tuple(key), n * es)
        self.full = self.buf.view(dtype, n).view(N, Dl + 2 * h, H, W, C)
        self.full.zero_()
        dc.group.barrier_host()          # nobody sends before every rank has cleared
        self.interior = self.full[:, h:h + Dl]
        self.h, self.dl = h, Dl
        r, P = dc.depth_rank, dc.depth_groups
        up, down = (r - 1 if r > 0 else None), (r + 1 if r < P - 1 else None)
        fl = dc._flags
        a = HaloSyncArgs()
        a.up_dst = self.buf.peer_ptr(up) if up is not None else None
        a.down_dst = self.buf.peer_ptr(down) if down is not None else None
        # my first planes land in the BOTTOM halo of the rank above, my last in the TOP halo below
        a.up_flag = fl.peer_ptr(up, (2 * slot + 1) * 4) if up is not None else None
        a.down_flag = fl.peer_ptr(down, (2 * slot) * 4) if down is not None else None
        a.top_flag = fl.ptr + (2 * slot) * 4 if up is not None else None
        a.bot_flag = fl.ptr + (2 * slot + 1) * 4 if down is not None else None
        a.local = dc._local_ctr.data_ptr() + 2 * slot * 4
        a.h = h
        self.args = a
        self.sent_bytes = N * h * H * W * C * es * ((up is not None) + (down is not None))

    def holds(self, t: torch.Tensor) -> bool:
        return (t.data_ptr() == self.interior.data_ptr() and t.shape == self.interior.shape
                and t.stride() == self.interior.stride())


class _DistConv(torch.autograd.Function):
    """Convolution of a depth-partitioned activation with the halo exchange inside the
    convolution kernels (forward and data gradient); see the module docstring.  Stands in
    for src/layers/learning/base_convolution.cpp:1355-1445."""

    @staticmethod
    def forward(ctx, x, w_leaf, b_leaf, dc: "DistconvContext", layer, h: int):
        from ..ops import native, nn
        from ..ops.conv import conv_fwd
        wh = layer.w.handle
        bh = layer.b.handle if layer.b is not None else None
        ksize, dil = tuple(layer.ksize), tuple(layer.dil)
        pad = (0,) + tuple(layer.pad[1:])
        act, act_p = layer.fused_act
        skip_act_grad = bool(getattr(layer, "skip_act_grad", False))
        x_cl = nn._cl_view(x)
        N, Dl, H, W, C = x_cl.shape
        Kout = wh.master.shape[0]
        ext = dc.halo_tensor(("x", layer.name), N, Dl, h, H, W, C, x.dtype)
        if not ext.holds(x_cl):
            ext.interior.copy_(x_cl)
            dc.interior_copies += 1
        nn._pack_both(wh, x.dtype, Kout, C, Kout, C, ksize)
        wt = wh.packed("fwd", x.dtype, lambda: nn.pack_filter(wh.master.detach(), x.dtype))
        bias = bh.master.detach() if bh is not None else None
        y = conv_fwd(ext.full, wt, ksize, pad=pad, stride=1, dilation=dil, bias=bias, act=act,
                     act_param=act_p, halo=ext.args)
        dc.halo_bytes += ext.sent_bytes
        layer._fused_halo = True
        layer._needs_dx = bool(ctx.needs_input_grad[0])
        ctx.save_for_backward(y if (act != native.ACT_NONE and not skip_act_grad) else None)
        ctx.meta = (dc, layer, h, ext, (N, Dl, H, W, C), Kout, act, act_p)
        return nn._from_cl(y, 5)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import nn
        from ..ops.conv import conv_fwd, conv_wgrad
        (y,) = ctx.saved_tensors
        dc, layer, h, ext, (N, Dl, H, W, C), Kout, act, act_p = ctx.meta
        wh = layer.w.handle
        bh = layer.b.handle if layer.b is not None else None
        ksize, dil = tuple(layer.ksize), tuple(layer.dil)
        pad = (0,) + tuple(layer.pad[1:])
        dy_cl = nn._cl_view(dy)
        Do, Ho, Wo = dy_cl.shape[1:4]
        dx = None
        if ctx.needs_input_grad[0]:
            dye = dc.halo_tensor(("dy", layer.name), N, Do, h, Ho, Wo, Kout, dy.dtype)
            if y is not None:
                dy_cl = nn._act_grad_from_output(y, dy_cl if dy_cl.is_contiguous() else dy_cl.contiguous(),
                                                 act, act_p)
            if not dye.holds(dy_cl):
                dye.interior.copy_(dy_cl)
                dc.interior_copies += 1
            dy_cl = dye.interior
            wt = wh.packed("dgrad", dy.dtype,
                           lambda: nn.pack_filter(wh.master.detach(), dy.dtype, for_dgrad=True))
            bpad = (0,) + tuple(d * (k - 1) - p for d, k, p in zip(dil[1:], ksize[1:], layer.pad[1:]))
            dx_cl = conv_fwd(dye.full, wt, ksize, pad=bpad, stride=1, dilation=dil,
                             out_dims=(Dl, H, W), halo=dye.args)
            dc.halo_bytes += dye.sent_bytes
            dx = nn._from_cl(dx_cl, 5)
        elif y is not None:
            dy_cl = nn._act_grad_from_output(y, dy_cl if dy_cl.is_contiguous() else dy_cl.contiguous(),
                                             act, act_p)
        if wh.grad is not None:
            # the extended input still holds the halo planes that forward received
            conv_wgrad(ext.full, dy_cl, ksize, pad=pad, stride=1, dilation=dil,
                       out=wh.grad.view(Kout, C, *ksize))
            wh.mark_ready()
        if bh is not None and bh.grad is not None:
            d2 = dy_cl if dy_cl.is_contiguous() else dy_cl.contiguous()
            bh.grad.add_(nn.column_sums(d2.reshape(-1, Kout)))
            bh.mark_ready()
        return dx, None, None, None, None, None


class _AllReduceSum(torch.autograd.Function):
    """Sum over the depth ranks; every rank then holds the full value, and only the
    depth-rank-0 copy carries the gradient weight back (the others would double count)."""

    @staticmethod
    def forward(ctx, t, dc):
        ctx.dc = dc
        out = t.float().contiguous().clone()
        dc.allreduce_depth_(out.view(-1))
        return out

    @staticmethod
    def backward(ctx, g):
        # d(total)/d(partial_r) = 1 on every rank; the loss itself is counted once per
        # sample group when the objective is formed (see DistconvContext.dist == SAMPLE rule).
        return g, None


class LineHaloExchange(torch.autograd.Function):
    """Halo exchange along one dimension of a depth x height x width grid.  x: logical
    [N, C, D, H, W]; ``dim`` = 2 (depth), 3 (height) or 4 (width); the result is 2h longer along it,
    with the neighbours' boundary slices at either end (``fill`` beyond the global
    boundary).  The ranks of the line through this rank trade their boundary slices with a
    library all-gather; backward sends the gradients of the received slices back and adds
    them to the owners' boundary."""

    @staticmethod
    def forward(ctx, x, dc: "DistconvContext", h: int, dim: int, fill: float = 0.0):
        P = (dc.depth_groups, dc.height_groups, dc.width_groups)[dim - 2]
        r = (dc.depth_rank, dc.height_rank, dc.width_rank)[dim - 2]
        L = x.shape[dim]
        ctx.meta = (dc, h, dim, P, r, L)
        lo, hi = x.narrow(dim, 0, h), x.narrow(dim, L - h, h)
        edges = torch.stack([lo, hi]).contiguous()
        allp = dc.comm.all_gather(edges, dc.line_pg[dim])
        shape = list(x.shape)
        shape[dim] = L + 2 * h
        xe = x.new_empty(shape)
        xe.narrow(dim, h, L).copy_(x)
        if r > 0:
            xe.narrow(dim, 0, h).copy_(allp[r - 1][1])
        else:
            xe.narrow(dim, 0, h).fill_(fill)
        if r < P - 1:
            xe.narrow(dim, h + L, h).copy_(allp[r + 1][0])
        else:
            xe.narrow(dim, h + L, h).fill_(fill)
        dc.halo_bytes += 2 * lo.numel() * lo.element_size()
        return xe

    @staticmethod
    def backward(ctx, gxe):
        dc, h, dim, P, r, L = ctx.meta
        edges = torch.stack([gxe.narrow(dim, 0, h), gxe.narrow(dim, h + L, h)]).contiguous()
        allp = dc.comm.all_gather(edges, dc.line_pg[dim])
        dx = gxe.narrow(dim, h, L).clone()
        if r > 0:             # what the rank before me computed for my first slices
            dx.narrow(dim, 0, h).add_(allp[r - 1][1])
        if r < P - 1:
            dx.narrow(dim, L - h, h).add_(allp[r + 1][0])
        return dx, None, None, None, None


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
        if dc.fused and P == g.world and r == g.rank:
            # interior copy, boundary fill, peer stores and both rendezvous in one launch
            xs = x_cl if x_cl.is_contiguous() else x_cl.contiguous()
            if g.halo_forward(xs, buf, N, Dl, h, plane, fill):
                dc.halo_bytes += 2 * N * h * plane
                return xe.permute(0, 4, 1, 2, 3)
        if dc.fused:
            raise native.NativeError("halo exchange: the tensor's planes are not multiples of "
                                     "16 bytes or it has fewer planes than the halo is wide")
        # host-side ranks (gloo): same data movement with a library all-gather
        xe[:, h:h + Dl].copy_(x_cl)
        if r == 0:
            xe[:, :h].fill_(fill)
        if r == P - 1:
            xe[:, h + Dl:].fill_(fill)
        edges = torch.stack([xe[:, h:2 * h], xe[:, Dl:Dl + h]]).contiguous()
        allp = dc.comm.all_gather(edges, dc.depth_pg)
        if r > 0:
            xe[:, :h].copy_(allp[r - 1][1])
        if r < P - 1:
            xe[:, h + Dl:].copy_(allp[r + 1][0])
        return xe.permute(0, 4, 1, 2, 3).clone()

    @staticmethod
    def backward(ctx, gxe):
        dc, h, tag, (N, C, Dl, H, W) = ctx.meta
        P, r = dc.depth_groups, dc.depth_rank
        g_cl = gxe.permute(0, 2, 3, 4, 1)
        if not g_cl.is_contiguous():
            g_cl = g_cl.contiguous()
        plane = H * W * C * g_cl.element_size()
        if not dc.fused:
            edges = torch.stack([g_cl[:, :h], g_cl[:, h + Dl:]]).contiguous()
            allp = dc.comm.all_gather(edges, dc.depth_pg)
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
        dx = torch.empty((N, Dl, H, W, C), dtype=g_cl.dtype, device=g_cl.device)
        if not (P == grp.world and r == grp.rank and grp.halo_backward(g_cl, buf, dx, N, Dl, h, plane)):
            raise native.NativeError("halo exchange (backward): the tensor's planes are not "
                                     "multiples of 16 bytes or it has fewer planes than the halo is wide")
        return dx.permute(0, 4, 1, 2, 3), None, None, None, None


class _Redistribute(torch.autograd.Function):
    """spatial -> sample (``to_sample=True``): rank r ends up with samples r, r+P, ... of the
    full depth extent; the inverse otherwise.  All-to-all by peer stores."""

    @staticmethod
    def forward(ctx, x, dc: DistconvContext, to_sample: bool, tag: str):
        out, total = _redistribute(x, dc, to_sample, tag + ("/s" if to_sample else "/p"))
        ctx.meta = (dc, to_sample, tag, total)
        return out

    @staticmethod
    def backward(ctx, g):
        dc, to_sample, tag, total = ctx.meta
        out, _ = _redistribute(g, dc, not to_sample, tag + ("/bs" if to_sample else "/bp"), total)
        return out, None, None, None


def _redistribute(x, dc: DistconvContext, to_sample: bool, tag: str, total=None):
    """Returns (tensor, number of samples of the sample group).  The samples of a group are
    dealt round-robin, so the last mini-batch of an epoch may leave the ranks with unequal
    (even zero) counts: towards the spatial layout every rank pads its share to the common
    maximum, and the padding is dropped where the bricks are put together."""
    if dc.channel_groups > 1:
        return _redistribute_channel(x, dc, to_sample, total)
    P, r = dc.depth_groups, dc.depth_rank
    x_cl = x.permute(0, 2, 3, 4, 1).contiguous()        # N, D, H, W, C
    es = x_cl.element_size()
    grp = dc.group
    S = dc.spatial_size
    if to_sample:
        total = x_cl.shape[0]
    else:
        if total is None:        # not known from a matching forward: ask the group
            cnt = torch.tensor([x_cl.shape[0]], dtype=torch.int64, device=x_cl.device)
            total = int(sum(int(c.item()) for c in dc.comm.all_gather(cnt, dc.depth_pg)))
        ns_max = (total + S - 1) // S
        if x_cl.shape[0] < ns_max:
            pad = x_cl.new_zeros((ns_max - x_cl.shape[0],) + tuple(x_cl.shape[1:]))
            x_cl = torch.cat([x_cl, pad], 0)
    out = _redistribute_cl(x_cl, dc, to_sample, tag, total, P, r, es, grp, S)
    return out, total


def _redistribute_channel(x, dc, to_sample: bool, total=None):
    """Channel (token) partition <-> sample-parallel for tensors [N, C, ...] of any rank."""
    S, sr = dc.channel_groups, dc.channel_rank
    x = x.contiguous()
    if to_sample:           # every rank's channel slice of all samples -> my samples, all channels
        total = x.shape[0]
        parts = dc.comm.all_gather(x, dc.depth_pg)
        return torch.cat([p[sr::S] for p in parts], dim=1), total
    if total is None:
        cnt = torch.tensor([x.shape[0]], dtype=torch.int64, device=x.device)
        total = int(sum(int(c.item()) for c in dc.comm.all_gather(cnt, dc.depth_pg)))
    ns_max = (total + S - 1) // S
    if x.shape[0] < ns_max:
        x = torch.cat([x, x.new_zeros((ns_max - x.shape[0],) + tuple(x.shape[1:]))], 0)
    parts = dc.comm.all_gather(x, dc.depth_pg)
    cl = x.shape[1] // S
    out = x.new_empty((total, cl) + tuple(x.shape[2:]))
    for q, part in enumerate(parts):
        out[q::S] = part[:len(range(q, total, S)), sr * cl:(sr + 1) * cl]
    return out, total


class _GatherChannels(torch.autograd.Function):
    """All ranks' channel slices of a [N, Cl, ...] tensor put together along dimension 1; the
    gradient of the local slice is the sum over the ranks of their gradients of it."""

    @staticmethod
    def forward(ctx, x, dc):
        ctx.dc = dc
        return torch.cat(dc.comm.all_gather(x.contiguous(), dc.depth_pg), dim=1)

    @staticmethod
    def backward(ctx, g):
        dc = ctx.dc
        g = g.contiguous().clone()
        dc.comm.allreduce(g, dc.depth_pg, "sum")
        cl = g.shape[1] // dc.channel_groups
        return g.narrow(1, dc.channel_rank * cl, cl).contiguous(), None


def _redistribute_cl(x_cl, dc, to_sample, tag, total, P, r, es, grp, S):
    if dc.grid_mode:
        # grid partition: every rank of the sample group contributes its brick
        Hg, Wg, S, sr = dc.height_groups, dc.width_groups, dc.spatial_size, dc.spatial_rank
        parts = dc.comm.all_gather(x_cl, dc.depth_pg)
        if to_sample:       # my samples (sr, sr + S, ...) of every brick, bricks put together
            out = torch.cat([torch.cat([torch.cat([parts[(d * Hg + i) * Wg + j][sr::S] for j in range(Wg)], dim=3)
                                        for i in range(Hg)], dim=2)
                             for d in range(P)], dim=1)
        else:               # my brick of every rank's samples, samples interleaved again
            ns, D, H, W = x_cl.shape[:4]
            Dl, Hl, Wl = D // P, H // Hg, W // Wg
            out = torch.empty((total, Dl, Hl, Wl) + tuple(x_cl.shape[4:]), dtype=x_cl.dtype, device=x_cl.device)
            for q, part in enumerate(parts):
                cq = len(range(q, total, S))
                out[q::S] = part[:cq, r * Dl:(r + 1) * Dl, dc.height_rank * Hl:(dc.height_rank + 1) * Hl,
                                 dc.width_rank * Wl:(dc.width_rank + 1) * Wl]
        return out.permute(0, 4, 1, 2, 3)
    if not dc.fused:
        parts = dc.comm.all_gather(x_cl, dc.depth_pg)
        if to_sample:
            out = torch.cat([p[r::P] for p in parts], dim=1)
        else:
            ns, D = x_cl.shape[0], x_cl.shape[1]
            Dl = D // P
            out = torch.empty((total, Dl) + tuple(x_cl.shape[2:]), dtype=x_cl.dtype, device=x_cl.device)
            for q, p in enumerate(parts):
                out[q::P] = p[:len(range(q, total, P)), r * Dl:(r + 1) * Dl]
        return out.permute(0, 4, 1, 2, 3)
    if to_sample:
        N, Dl, H, W, C = x_cl.shape
        ns = (N + P - 1) // P                           # samples per rank (round-robin owner)
        slab = Dl * H * W * C * es
        buf = dc.buffer(("redist", tag), ns * P * slab)
        mine = len(range(r, N, P))
        view = buf.view(x_cl.dtype, ns * P * Dl * H * W * C).view(ns, P * Dl, H, W, C)
        # sample n, depth slab r -> slot [n // P][r] of owner n % P: one kernel, one rendezvous;
        # the result is read where it landed (two uses of the buffer are a training step apart)
        if grp.alltoall_slabs(x_cl, buf, N, slab):
            return view[:mine].permute(0, 4, 1, 2, 3)
        for q in range(P):
            rows = x_cl[q::P]
            if rows.shape[0] == 0:
                continue
            grp.put_rows(rows, buf, q, r * slab, rows.shape[0], slab, P * slab, P * slab)
        grp.barrier_device(3)
        out = view[:mine].clone()
        grp.barrier_device(2)
        return out.permute(0, 4, 1, 2, 3)
    ns, D, H, W, C = x_cl.shape
    Dl = D // P
    slab = Dl * H * W * C * es
    # every rank brings ns samples (shares padded to the common maximum by the caller); rows
    # beyond ``total`` are that padding
    N = ns * P
    buf = dc.buffer(("redist", tag), N * slab)
    view = buf.view(x_cl.dtype, N * Dl * H * W * C).view(N, Dl, H, W, C)
    # my sample j (global index j * P + r), depth slab q -> row j * P + r of rank q's buffer
    if grp.alltoall_slabs(x_cl, buf, ns * P, slab):
        return view[:total].permute(0, 4, 1, 2, 3)
    for q in range(P):
        src = x_cl[:, q * Dl:(q + 1) * Dl]
        grp.put_rows(src, buf, q, r * slab, ns, slab, D * H * W * C * es, P * slab)
    grp.barrier_device(3)
    out = view[:total].clone()
    grp.barrier_device(2)
    return out.permute(0, 4, 1, 2, 3)
