"""Executable layers: transform, math, misc and image families.

Most of these are data-movement or small reductions; they are composed from PyTorch
tensor operations (differentiated by autograd) and keep the reference's shapes and
conventions.  Reference sources: include/lbann/layers/transform/*.hpp,
src/layers/transform/*.cu, src/layers/misc/*.cu, src/layers/math/*.cpp,
src/layers/image/*.cu.
"""
from __future__ import annotations

import importlib.util
import math
from typing import List

import torch
import torch.nn.functional as F

from ..ops import native, nn
from ..ops import elementwise as ew
from ..ops.gemm import gemm
from .layer_base import ExecLayer, broadcast_list, prod, register, rows2d


# =============================================================================== shape / routing
@register("reshape")
class Reshape(ExecLayer):
    """View with new per-sample dims; one entry may be -1 (include/lbann/layers/transform/reshape.hpp)."""

    def setup(self, in_dims):
        dims = [int(d) for d in self.params.dims]
        if self.hint_layer and not dims:
            dims = list(self.model.layer(self.hint_layer).out_dims[0])
        total = prod(in_dims[0])
        if -1 in dims:
            known = prod([d for d in dims if d != -1])
            dims[dims.index(-1)] = total // max(known, 1)
        if prod(dims) != total:
            raise ValueError(f"{self.name}: cannot reshape {in_dims[0]} to {dims}")
        return [tuple(dims)]

    def forward(self, xs, training):
        return [xs[0].reshape(xs[0].shape[0], *self.out_dims[0])]


@register("split")
class Split(ExecLayer):
    """Same tensor to every child (include/lbann/layers/transform/split.hpp)."""
    num_outputs = -1
    supports_distconv = True

    def setup(self, in_dims):
        return [tuple(in_dims[0])] * max(1, len(self.child_names))

    def forward(self, xs, training):
        return [xs[0]] * max(1, len(self.child_names))


@register("sum")
class Sum(ExecLayer):
    supports_channel_parallel = True
    """Entrywise sum of all inputs (include/lbann/layers/transform/sum.hpp)."""
    max_parents = -1
    supports_distconv = True

    def forward(self, xs, training):
        xs = [self.cast_in(x) for x in xs]
        out = xs[0]
        relu = getattr(self, "fused_act", (native.ACT_NONE, 0.0))[0] == native.ACT_RELU
        for k, x in enumerate(xs[1:]):
            if relu and k == len(xs) - 2:        # the ReLU that follows rides on the last addition
                out = ew.add_relu(out, x.reshape(out.shape))
                relu = False
            else:
                out = ew.binary("add", out, x.reshape(out.shape))
        if relu:
            out = torch.relu(out)
        return [out]


@register("weighted_sum")
class WeightedSum(ExecLayer):
    supports_channel_parallel = True
    max_parents = -1

    def forward(self, xs, training):
        f = list(self.params.scaling_factors) or [1.0] * len(xs)
        out = None
        for s, x in zip(f, xs):
            t = self.cast_in(x) * s
            out = t if out is None else out + t.reshape(out.shape)
        return [out]


@register("hadamard")
class Hadamard(ExecLayer):
    supports_channel_parallel = True
    max_parents = -1

    def forward(self, xs, training):
        out = self.cast_in(xs[0])
        for x in xs[1:]:
            out = ew.binary("multiply", out, self.cast_in(x).reshape(out.shape))
        return [out]


@register("concatenation")
class Concatenation(ExecLayer):
    """Concatenate along a sample axis (src/layers/transform/concatenate.cu)."""
    max_parents = -1
    supports_distconv = True

    def setup(self, in_dims):
        self.axis = int(self.params.axis)
        if self.axis < 0:
            self.axis += len(in_dims[0])
        d = list(in_dims[0])
        d[self.axis] = sum(int(x[self.axis]) for x in in_dims)
        return [tuple(d)]

    def forward(self, xs, training):
        return [torch.cat([self.cast_in(x) for x in xs], dim=self.axis + 1)]


@register("slice")
class Slice(ExecLayer):
    """Split along an axis at ``slice_points`` (src/layers/transform/slice.cu)."""
    num_outputs = -1
    supports_distconv = True

    def setup(self, in_dims):
        p = self.params
        self.axis = int(p.axis)
        if self.axis < 0:
            self.axis += len(in_dims[0])
        pts = [int(v) for v in p.slice_points]
        if p.get_slice_points_from_reader:
            pts = self.model.slice_points_from_reader(p.get_slice_points_from_reader)
        self.points = pts
        outs = []
        for a, b in zip(pts[:-1], pts[1:]):
            d = list(in_dims[0])
            d[self.axis] = b - a
            outs.append(tuple(d))
        return outs

    def forward(self, xs, training):
        x = xs[0]
        return [x.narrow(self.axis + 1, a, b - a) for a, b in zip(self.points[:-1], self.points[1:])]


@register("permute")
class TensorPermute(ExecLayer):
    """Permute the sample dims (src/layers/transform/permute.cpp)."""

    def setup(self, in_dims):
        self.axes = [int(a) for a in self.params.axes]
        return [tuple(in_dims[0][a] for a in self.axes)]

    def forward(self, xs, training):
        return [xs[0].permute(0, *[a + 1 for a in self.axes])]


@register("crop")
class Crop(ExecLayer):
    """Crop a window of ``dims``; the second input gives the normalised position in [0,1]
    of the window along every dim (src/layers/transform/crop.cu)."""
    min_parents = max_parents = 2

    def setup(self, in_dims):
        return [tuple(int(d) for d in self.params.dims)]

    def forward(self, xs, training):
        x, pos = xs[0], rows2d(xs[1]).float()
        out_d, in_d = self.out_dims[0], self.in_dims[0]
        outs = []
        for n in range(x.shape[0]):
            sl = [n]
            for k, (o, i) in enumerate(zip(out_d, in_d)):
                off = int(torch.round(pos[n, k] * (i - o)).item())
                off = max(0, min(off, i - o))
                sl.append(slice(off, off + o))
            outs.append(x[tuple(sl)])
        return [torch.stack(outs)]


@register("tessellate")
class Tessellate(ExecLayer):
    """Tile the input periodically to fill ``dims`` (src/layers/transform/tessellate.cu)."""

    def setup(self, in_dims):
        dims = [int(d) for d in self.params.dims]
        if self.hint_layer and not dims:
            dims = list(self.model.layer(self.hint_layer).out_dims[0])
        return [tuple(dims)]

    def forward(self, xs, training):
        x = xs[0]
        ind, outd = self.in_dims[0], self.out_dims[0]
        ind = (1,) * (len(outd) - len(ind)) + tuple(ind)
        x = x.reshape(x.shape[0], *ind)
        reps = [1] + [-(-o // i) for o, i in zip(outd, ind)]
        y = x.repeat(*reps)
        return [y[(slice(None),) + tuple(slice(0, o) for o in outd)]]


@register("upsample")
class Upsample(ExecLayer):
    """Nearest-neighbour upsampling by integer factors (src/layers/transform/upsample.cpp)."""
    supports_distconv = True

    def setup(self, in_dims):
        p = self.params
        nd = int(p.num_dims) or (len(in_dims[0]) - 1)
        self.factors = broadcast_list(p.scale_factors, nd, 1) if p.has_vectors or len(p.scale_factors) \
            else (int(p.scale_factors_i) or 1,) * nd
        d = in_dims[0]
        return [(d[0],) + tuple(s * f for s, f in zip(d[1:], self.factors))]

    def forward(self, xs, training):
        x = xs[0]
        for ax, f in enumerate(self.factors):
            if f != 1:
                x = x.repeat_interleave(f, dim=ax + 2)
        return [x]


@register("pooling")
class Pooling(ExecLayer):
    """Max / average pooling (src/layers/transform/pooling.cpp:111-176)."""
    supports_distconv = True
    supports_channel_parallel = True

    def setup(self, in_dims):
        p = self.params
        nd = int(p.num_dims) or (len(in_dims[0]) - 1)
        if p.has_vectors or len(p.pool_dims):
            self.k = broadcast_list(p.pool_dims, nd, 1)
            self.pad = broadcast_list(p.pool_pads, nd, 0)
            self.stride = broadcast_list(p.pool_strides, nd, 1)
        else:
            self.k = (int(p.pool_dims_i) or 1,) * nd
            self.pad = (int(p.pool_pads_i),) * nd
            self.stride = (int(p.pool_strides_i) or 1,) * nd
        self.mode = p.pool_mode or "max"
        d = in_dims[0]
        sp = tuple((i + 2 * pd - k) // s + 1 for i, pd, k, s in zip(d[1:], self.pad, self.k, self.stride))
        return [(d[0],) + sp]

    def forward(self, xs, training):
        if getattr(self, "input_is_pooled", False):
            # the producing first-layer convolution ran this pooling inside its own kernel
            self.input_is_pooled = False
            return [xs[0]]
        x = self.cast_in(xs[0])
        dc = self.model.distconv
        if dc is not None and dc.enabled(self):
            return [dc.pooling(self, x)]
        act = getattr(self, "bwd_act", (0, 0.0))
        return [nn.pooling(x, self.k, self.pad, self.stride, self.mode, act[0], act[1])]


@register("unpooling")
class Unpooling(ExecLayer):
    """Inverse of the max pooling layer named by ``hint_layer``: values go back to the
    arg-max positions (include/lbann/layers/transform/unpooling.hpp)."""

    def setup(self, in_dims):
        self.pool = self.model.layer(self.hint_layer)
        return [tuple(self.pool.in_dims[0])]

    def forward(self, xs, training):
        pool = self.pool
        src = self.model.activation(pool.parent_names[0])
        nsp = src.dim() - 2
        fn = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nsp]
        with torch.no_grad():
            _, idx = fn(src.float(), pool.k, pool.stride, pool.pad, return_indices=True)
        un = {1: F.max_unpool1d, 2: F.max_unpool2d, 3: F.max_unpool3d}[nsp]
        return [un(xs[0].float(), idx, pool.k, pool.stride, pool.pad, src.shape[2:]).to(xs[0].dtype)]


# =============================================================================== generators
class _Generator(ExecLayer):
    min_parents = 0
    max_parents = 1

    def _dims(self):
        dims = [int(d) for d in self.params.neuron_dims]
        if self.hint_layer and not dims:
            dims = list(self.model.layer(self.hint_layer).out_dims[0])
        return tuple(dims) or (1,)

    def setup(self, in_dims):
        return [self._dims()]

    def _shape(self):
        return (self.model.current_mini_batch_size,) + self.out_dims[0]

    def _opts(self):
        return dict(device=self.model.device, dtype=self.dtype or self.model.default_dtype)


@register("constant")
class Constant(_Generator):
    def _dims(self):
        dims = [int(d) for d in self.params.num_neurons]
        if self.hint_layer and not dims:
            dims = list(self.model.layer(self.hint_layer).out_dims[0])
        return tuple(dims) or (1,)

    def forward(self, xs, training):
        return [torch.full(self._shape(), float(self.params.value), **self._opts())]


@register("gaussian")
class Gaussian(_Generator):
    def forward(self, xs, training):
        p = self.params
        if p.training_only and not training:
            return [torch.full(self._shape(), float(p.mean), **self._opts())]
        sd = float(p.stdev) if (p.stdev or p.mean) else 1.0
        g = torch.randn(self._shape(), device=self.model.device, generator=self.model.generator())
        return [(g * sd + float(p.mean)).to(self._opts()["dtype"])]


@register("uniform")
class Uniform(_Generator):
    def forward(self, xs, training):
        p = self.params
        lo, hi = float(p.min), float(p.max)
        if lo == 0.0 and hi == 0.0:
            hi = 1.0
        if p.training_only and not training:
            return [torch.full(self._shape(), 0.5 * (lo + hi), **self._opts())]
        u = torch.rand(self._shape(), device=self.model.device, generator=self.model.generator())
        return [(u * (hi - lo) + lo).to(self._opts()["dtype"])]


@register("bernoulli")
class Bernoulli(_Generator):
    def forward(self, xs, training):
        u = torch.rand(self._shape(), device=self.model.device, generator=self.model.generator())
        return [(u < (float(self.params.prob) or 0.5)).to(self._opts()["dtype"])]


@register("categorical_random")
class CategoricalRandom(ExecLayer):
    """One-hot sample from the input probabilities during training, arg-max otherwise."""

    def forward(self, xs, training):
        p = rows2d(xs[0]).float()
        idx = torch.multinomial(p.clamp(min=0) + 1e-30, 1).squeeze(1) if training else p.argmax(1)
        return [F.one_hot(idx, p.shape[1]).to(xs[0].dtype).reshape(xs[0].shape)]


@register("discrete_random")
class DiscreteRandom(ExecLayer):
    def setup(self, in_dims):
        self.values = torch.tensor(list(self.params.values), dtype=torch.float32)
        return [tuple(int(d) for d in self.params.dims) or (1,)]

    def forward(self, xs, training):
        p = rows2d(xs[0]).float()
        n = prod(self.out_dims[0])
        if training:
            idx = torch.multinomial(p.clamp(min=0) + 1e-30, n, replacement=True)
            out = self.values.to(p.device)[idx]
        else:
            out = (p * self.values.to(p.device)).sum(1, keepdim=True).expand(-1, n)
        return [out.reshape(p.shape[0], *self.out_dims[0]).to(xs[0].dtype)]


@register("weights_layer")
class WeightsLayer(ExecLayer):
    """Outputs a weights tensor, replicated over the mini-batch."""
    min_parents = max_parents = 0

    def setup(self, in_dims):
        dims = tuple(int(d) for d in self.params.dims)
        self.w = self.get_weights(0, "weights", dims)
        return [dims]

    def forward(self, xs, training):
        w = self.w.handle.master.to(self.dtype or self.model.default_dtype)
        return [w.unsqueeze(0).expand(self.model.current_mini_batch_size, *w.shape)]


@register("mini_batch_index")
class MiniBatchIndex(ExecLayer):
    min_parents = max_parents = 0

    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        n = self.model.current_mini_batch_size
        off = self.model.mini_batch_offset()
        return [(torch.arange(n, device=self.model.device, dtype=torch.float32) + off).reshape(n, 1)]


@register("mini_batch_size")
class MiniBatchSize(ExecLayer):
    min_parents = max_parents = 0

    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        n = self.model.current_mini_batch_size
        g = self.model.global_mini_batch_size()
        return [torch.full((n, 1), float(g), device=self.model.device)]


# =============================================================================== reductions
@register("reduction")
class Reduction(ExecLayer):
    """Sum or mean of each sample (include/lbann/layers/transform/reduction.hpp)."""

    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        x = rows2d(self.cast_in(xs[0]))
        mode = (self.params.mode or "sum").lower()
        r = x.float().sum(1, keepdim=True)
        if mode in ("mean", "average"):
            r = r / x.shape[1]
        return [r.to(x.dtype)]


@register("multidim_reduction")
class MultiDimReduction(ExecLayer):
    def setup(self, in_dims):
        self.axes = sorted(int(a) for a in self.params.axes)
        d = [s for i, s in enumerate(in_dims[0]) if i not in self.axes]
        return [tuple(d) or (1,)]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        mode = (self.params.mode or "sum").lower()
        dims = [a + 1 for a in self.axes]
        r = x.float().sum(dims) if mode == "sum" else (x.float().amax(dims) if mode == "max" else x.float().mean(dims))
        return [r.reshape(x.shape[0], *self.out_dims[0]).to(x.dtype)]


@register("batchwise_reduce_sum")
class BatchwiseReduceSum(ExecLayer):
    """Sum over the (global) mini-batch, replicated to every sample."""

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        s = x.float().sum(0, keepdim=True)
        par = self.model.parallel
        if par is not None and par.dp_size > 1:
            s = nn._ReduceSum.apply(s, par.allreduce_sum_inplace)
        return [s.expand_as(x).to(x.dtype)]


@register("channelwise_mean")
class ChannelwiseMean(ExecLayer):
    def setup(self, in_dims):
        return [(int(in_dims[0][0]),)]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        return [x.reshape(x.shape[0], x.shape[1], -1).float().mean(2).to(x.dtype)]


@register("variance")
class Variance(ExecLayer):
    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        x = rows2d(self.cast_in(xs[0])).float()
        n = x.shape[1]
        v = ((x - x.mean(1, keepdim=True)) ** 2).sum(1, keepdim=True)
        return [(v / (n if self.params.biased else max(n - 1, 1))).to(xs[0].dtype)]


@register("covariance")
class Covariance(ExecLayer):
    min_parents = max_parents = 2

    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        a = rows2d(self.cast_in(xs[0])).float()
        b = rows2d(self.cast_in(xs[1])).float()
        n = a.shape[1]
        c = ((a - a.mean(1, keepdim=True)) * (b - b.mean(1, keepdim=True))).sum(1, keepdim=True)
        return [(c / (n if self.params.biased else max(n - 1, 1))).to(xs[0].dtype)]


@register("argmax")
class Argmax(ExecLayer):
    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        x = rows2d(xs[0])
        return [x.argmax(1, keepdim=True).to(xs[0].dtype)]


@register("argmin")
class Argmin(ExecLayer):
    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        x = rows2d(xs[0])
        return [x.argmin(1, keepdim=True).to(xs[0].dtype)]


@register("one_hot")
class OneHot(ExecLayer):
    """Index -> one-hot vector of ``size``; out-of-range gives zeros (src/layers/misc/one_hot.cu)."""

    def setup(self, in_dims):
        self.size = int(self.params.size)
        return [(self.size,)]

    def forward(self, xs, training):
        idx = xs[0].reshape(-1).long()
        ok = (idx >= 0) & (idx < self.size)
        out = F.one_hot(idx.clamp(0, self.size - 1), self.size) * ok[:, None]
        return [out.to(self.dtype or self.model.default_dtype)]


@register("in_top_k")
class InTopK(ExecLayer):
    """1 for the k largest entries of each sample, else 0 (src/layers/transform/in_top_k.cu)."""

    def forward(self, xs, training):
        x = rows2d(xs[0])
        k = min(int(self.params.k), x.shape[1])
        out = torch.zeros_like(x)
        if k > 0:
            idx = x.float().topk(k, dim=1).indices
            out.scatter_(1, idx, 1.0)
        return [out.reshape(xs[0].shape)]


@register("sort")
class Sort(ExecLayer):
    def forward(self, xs, training):
        x = rows2d(xs[0])
        y, _ = torch.sort(x, dim=1, descending=bool(self.params.descending))
        return [y.reshape(xs[0].shape)]


# =============================================================================== gather / scatter
@register("gather")
class Gather(ExecLayer):
    """out[..., j, ...] = values[..., ind[j], ...] along ``axis`` (default 0); out-of-range
    indices give zeros (src/layers/transform/gather.cu)."""
    min_parents = max_parents = 2
    supports_distconv = True

    def setup(self, in_dims):
        v, ind = in_dims[0], in_dims[1]
        self.axis = int(self.params.axis.value) if self.params.HasField("axis") else 0
        if len(v) == 1:
            return [tuple(ind)]
        d = list(v)
        d[self.axis] = prod(ind)
        return [tuple(d)]

    def forward(self, xs, training):
        v = self.cast_in(xs[0])
        n = v.shape[0]
        ind = rows2d(xs[1]).long()
        if v.dim() == 2:
            ok = (ind >= 0) & (ind < v.shape[1])
            out = v.gather(1, ind.clamp(0, v.shape[1] - 1)) * ok.to(v.dtype)
            return [out.reshape(n, *self.out_dims[0])]
        ax = self.axis + 1
        size = v.shape[ax]
        ok = (ind >= 0) & (ind < size)
        shape = [n] + [1] * (v.dim() - 1)
        shape[ax] = ind.shape[1]
        idx = ind.clamp(0, size - 1).reshape(shape).expand(*[ind.shape[1] if i == ax else s
                                                           for i, s in enumerate(v.shape)])
        out = v.gather(ax, idx) * ok.reshape(shape).to(v.dtype)
        return [out]


@register("scatter")
class Scatter(ExecLayer):
    """out[ind[j]] += values[j] along ``axis`` into a tensor of ``dims``
    (src/layers/transform/scatter.cu)."""
    min_parents = max_parents = 2
    supports_distconv = True

    def setup(self, in_dims):
        self.axis = int(self.params.axis.value) if self.params.HasField("axis") else 0
        return [tuple(int(d) for d in self.params.dims)]

    def forward(self, xs, training):
        v = self.cast_in(xs[0])
        n = v.shape[0]
        ind = rows2d(xs[1]).long()
        outd = self.out_dims[0]
        if len(outd) == 1:
            size = outd[0]
            ok = (ind >= 0) & (ind < size)
            out = torch.zeros(n, size, dtype=v.dtype, device=v.device)
            out = out.scatter_add(1, ind.clamp(0, size - 1), rows2d(v) * ok.to(v.dtype))
            return [out]
        ax = self.axis + 1
        size = outd[self.axis]
        ok = (ind >= 0) & (ind < size)
        shape = [n] + [1] * (v.dim() - 1)
        shape[ax] = ind.shape[1]
        idx = ind.clamp(0, size - 1).reshape(shape).expand_as(v)
        out = torch.zeros(n, *outd, dtype=v.dtype, device=v.device)
        out = out.scatter_add(ax, idx, v * ok.reshape(shape).to(v.dtype))
        return [out]


# =============================================================================== math
@register("matmul")
class MatMul(ExecLayer):
    supports_channel_parallel = True
    """Per-sample matrix product of two (batched) 2-D inputs with optional transposes
    (src/layers/math/matmul.cpp:419-584)."""
    min_parents = max_parents = 2
    supports_distconv = True

    def setup(self, in_dims):
        a, b = in_dims
        self.ta, self.tb = bool(self.params.transpose_a), bool(self.params.transpose_b)
        m = a[-1] if self.ta else a[-2]
        n = b[-2] if self.tb else b[-1]
        return [tuple(a[:-2]) + (m, n)]

    def forward(self, xs, training):
        a, b = self.cast_in(xs[0]), self.cast_in(xs[1])
        dc = self.model.distconv
        if dc is not None and dc.channel_groups > 1 and dc.enabled(self):
            # rows of the first operand stay with their rank; the second operand is needed whole
            if self.ta:
                raise NotImplementedError("a channel-partitioned matrix product cannot transpose its first operand")
            b = dc.gather_channels(b)
        if a.is_cuda and a.dtype in (torch.float16, torch.bfloat16):
            return [_BatchedMatMul.apply(a, b.to(a.dtype), self.ta, self.tb)]
        A = a.transpose(-1, -2) if self.ta else a
        B = b.transpose(-1, -2) if self.tb else b
        return [A @ B]


class _BatchedMatMul(torch.autograd.Function):
    """Strided-batched tcgen05 GEMM with analytic gradients (no transposes materialised)."""

    @staticmethod
    def forward(ctx, a, b, ta, tb):
        ctx.save_for_backward(a, b)
        ctx.meta = (ta, tb)
        a3 = a.reshape(-1, *a.shape[-2:]).contiguous()
        b3 = b.reshape(-1, *b.shape[-2:]).contiguous()
        y = gemm(a3, b3, trans_a=ta, trans_b=tb)
        return y.reshape(*a.shape[:-2], *y.shape[-2:])

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        ta, tb = ctx.meta
        a3 = a.reshape(-1, *a.shape[-2:]).contiguous()
        b3 = b.reshape(-1, *b.shape[-2:]).contiguous()
        g = dy.reshape(-1, *dy.shape[-2:]).contiguous()
        # C = op(A) op(B)
        if not ta:
            da = gemm(g, b3, trans_b=not tb)            # dA = dC op(B)^T
        else:
            da = gemm(b3, g, trans_a=tb, trans_b=True)  # dA^T... A stored [K,M]: dA = op(B) dC^T
        if not tb:
            db = gemm(a3, g, trans_a=not ta)            # dB = op(A)^T dC
        else:
            db = gemm(g, a3, trans_a=True, trans_b=ta)  # B stored [N,K]: dB = dC^T op(A)
        return da.reshape(a.shape), db.reshape(b.shape), None, None


@register("dft_abs")
class DFTAbs(ExecLayer):
    """|DFT| over the spatial dims of every channel (src/layers/misc/dft_abs.cu)."""

    def forward(self, xs, training):
        x = xs[0].float()
        dims = tuple(range(2, x.dim()))
        return [torch.fft.fftn(x, dim=dims).abs().to(xs[0].dtype)]


# =============================================================================== misc
@register("channelwise_softmax")
class ChannelwiseSoftmax(ExecLayer):
    supports_channel_parallel = True
    """Softmax within each channel (row) of the sample; with ``single_dim_mode`` only along
    ``dim`` (src/layers/misc/channelwise_softmax.cu:238-319)."""

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        p = self.params
        scale, causal = getattr(self, "fused_scale", 1.0), getattr(self, "fused_causal", 0)
        if p.single_dim_mode:
            dim = int(p.dim)
            if dim < 0:
                dim += len(self.in_dims[0])
            if dim == len(self.in_dims[0]) - 1:
                return [nn.softmax_lastdim(x, False, scale, causal)]
            xm = x.movedim(dim + 1, -1)
            return [nn.softmax_lastdim(xm.contiguous(), False, scale, causal).movedim(-1, dim + 1)]
        n, c = x.shape[0], x.shape[1]
        return [nn.softmax_lastdim(x.reshape(n, c, -1), False, scale, causal).reshape(x.shape)]


@register("stop_gradient")
class StopGradient(ExecLayer):
    def forward(self, xs, training):
        return [xs[0].detach()]


@register("dummy")
class Dummy(ExecLayer):
    num_outputs = 0

    def setup(self, in_dims):
        return []

    def forward(self, xs, training):
        return []


@register("evaluation")
class Evaluation(ExecLayer):
    """Marks a scalar-per-sample tensor for the objective / metrics; the model reads the
    mean over the global mini-batch (src/layers/transform/evaluation.cpp:49-82)."""
    num_outputs = 0

    def setup(self, in_dims):
        return []

    def forward(self, xs, training):
        return []


@register("identity_zero")
class IdentityZero(ExecLayer):
    """The input while the layer is unfrozen, zeros (and no gradient) while it is frozen: the
    switch on each side's loss in alternating GAN updates
    (src/layers/transform/identity_zero.cpp:66-90)."""

    def forward(self, xs, training):
        if self.frozen:
            return [torch.zeros_like(xs[0])]
        return [xs[0]]


@register("uniform_hash")
class UniformHash(ExecLayer):
    """Deterministic hash of each entry to [0, 1) (src/layers/misc/uniform_hash.cu)."""

    def forward(self, xs, training):
        x = xs[0].float()
        bits = x.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        h = bits
        h = ((h ^ (h >> 16)) * 0x85EBCA6B) & 0xFFFFFFFF
        h = ((h ^ (h >> 13)) * 0xC2B2AE35) & 0xFFFFFFFF
        h = h ^ (h >> 16)
        return [(h.float() / 4294967296.0).to(xs[0].dtype)]


@register("rowwise_weights_norms")
class RowwiseWeightsNorms(ExecLayer):
    """L2 norm of every row of a weights matrix (src/layers/misc/rowwise_weights_norms.cu)."""
    min_parents = max_parents = 0

    def setup(self, in_dims):
        self.w = self.model.weights_by_name[self.weight_names[0]]
        self.w.users.append(self)
        self.weights = [self.w]
        return [(int(self.w.shape[0]),)]

    def forward(self, xs, training):
        w = self.w.handle.master
        norms = rows2d(w).float().norm(dim=1)
        return [norms.unsqueeze(0).expand(self.model.current_mini_batch_size, -1)]


@register("dist_embedding")
class DistEmbedding(ExecLayer):
    """Embedding table partitioned over ranks with peer access to remote rows and an
    optional built-in sparse SGD (src/layers/misc/dist_embedding.cu).  Rows are fetched
    from the owning rank through the communicator's peer-memory gather."""

    def setup(self, in_dims):
        p = self.params
        self.num, self.dim = int(p.num_embeddings), int(p.embedding_dim)

        def init(shape, gen, fi, fo):
            return torch.randn(self.dim * self.num, generator=gen)
        self.w = self.get_weights(0, "weights", (self.num, self.dim), init,
                                  optimizer=not bool(p.sparse_sgd))
        return [tuple(in_dims[0]) + (self.dim,)]

    def forward(self, xs, training):
        idx = xs[0].long()
        par = self.model.parallel
        if self.params.sparse_sgd:
            # built-in sparse SGD; with several ranks the table is partitioned and rows are
            # accessed one-sidedly (replicated on host-side ranks)
            from ..parallel.dist_embedding import dist_embedding
            return [dist_embedding(par, self, idx, training)]
        ok = (idx >= 0) & (idx < self.num)
        table = self.w.handle.master
        out = F.embedding(idx.clamp(0, self.num - 1), table) * ok.unsqueeze(-1)
        return [out.to(self.dtype or self.model.default_dtype)]


@register("external")
class External(ExecLayer):
    """User-supplied layer loaded at run time.  The reference dlopens a C++ shared object
    (include/lbann/layers/misc/external.hpp); here ``filename`` may be a Python file (or a
    shared object exposing a Python-importable module) defining ``layer_name`` as a class
    with ``setup(in_dims) -> out_dims`` and ``forward(xs, training) -> ys``."""
    max_parents = -1

    def setup(self, in_dims):
        spec = importlib.util.spec_from_file_location("lbann_external_" + self.name, self.params.filename)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        self.impl = getattr(mod, self.params.layer_name or "Layer")()
        return [tuple(d) for d in self.impl.setup(in_dims)]

    def forward(self, xs, training):
        return list(self.impl.forward(xs, training))


# =============================================================================== image
@register("bilinear_resize")
class BilinearResize(ExecLayer):
    """src/layers/image/bilinear_resize.cu"""

    def setup(self, in_dims):
        d = in_dims[0]
        return [tuple(d[:-2]) + (int(self.params.height), int(self.params.width))]

    def forward(self, xs, training):
        x = xs[0]
        lead = x.shape[:-2]
        y = F.interpolate(x.reshape(-1, 1, *x.shape[-2:]).float(), size=self.out_dims[0][-2:],
                          mode="bilinear", align_corners=False)
        return [y.reshape(*lead, *self.out_dims[0][-2:]).to(x.dtype)]


def _affine_sample(img, theta):
    grid = F.affine_grid(theta, img.shape, align_corners=False)
    return F.grid_sample(img, grid, mode="bilinear", padding_mode="zeros", align_corners=False)


@register("rotation")
class Rotation(ExecLayer):
    """Rotate each image counter-clockwise by the angle (degrees) in the second input
    (src/layers/image/rotation.cpp)."""
    min_parents = max_parents = 2

    def forward(self, xs, training):
        img = xs[0].float()
        ang = xs[1].reshape(-1).float() * math.pi / 180.0
        c, s = torch.cos(ang), torch.sin(ang)
        z = torch.zeros_like(c)
        theta = torch.stack([torch.stack([c, -s, z], 1), torch.stack([s, c, z], 1)], 1)
        return [_affine_sample(img, theta).to(xs[0].dtype)]


@register("composite_image_transformation")
class CompositeImageTransformation(ExecLayer):
    """Rotation, shear and translation in one resampling pass
    (src/layers/image/composite_image_transformation.cpp).  Inputs: image, rotation angle
    (degrees), shear (x, y), translation (x, y) in pixels."""
    min_parents = max_parents = 4

    def forward(self, xs, training):
        img = xs[0].float()
        n, _, H, W = img.shape
        ang = xs[1].reshape(-1).float() * math.pi / 180.0
        sh = xs[2].reshape(n, 2).float()
        tr = xs[3].reshape(n, 2).float()
        c, s = torch.cos(ang), torch.sin(ang)
        a00 = c + (-s) * sh[:, 1]
        a01 = c * sh[:, 0] - s
        a10 = s + c * sh[:, 1]
        a11 = s * sh[:, 0] + c
        theta = torch.stack([torch.stack([a00, a01, -2 * tr[:, 0] / W], 1),
                             torch.stack([a10, a11, -2 * tr[:, 1] / H], 1)], 1)
        return [_affine_sample(img, theta).to(xs[0].dtype)]


@register("cutout")
class Cutout(ExecLayer):
    """Zero a square window of each image; inputs: image, centre (normalised x, y), side
    length in pixels (src/layers/image/cutout.cpp)."""
    min_parents = max_parents = 3

    def forward(self, xs, training):
        img = xs[0]
        n, _, H, W = img.shape
        ctr = xs[1].reshape(n, 2).float()
        side = xs[2].reshape(n).float()
        yy = torch.arange(H, device=img.device).view(1, H, 1).float()
        xx = torch.arange(W, device=img.device).view(1, 1, W).float()
        cx, cy = (ctr[:, 0] * W).view(n, 1, 1), (ctr[:, 1] * H).view(n, 1, 1)
        half = (side / 2).view(n, 1, 1)
        inside = ((xx - cx).abs() <= half) & ((yy - cy).abs() <= half)
        return [img * (~inside).unsqueeze(1).to(img.dtype)]


# =============================================================================== sub-graph collectives
@register("cross_grid_sum")
class CrossGridSum(ExecLayer):
    """Sum of the same tensor across sub-grids; every branch gets the total
    (include/lbann/layers/transform/cross_grid_sum.hpp:113-148)."""
    max_parents = -1
    num_outputs = -1

    def setup(self, in_dims):
        return [tuple(d) for d in in_dims]

    def forward(self, xs, training):
        # With sub-grids the executor has brought every branch's tensor to this layer's grid
        # (the whole trainer, since its parents sit on different grids) and sends the total
        # back out to the branches; the layer itself is a plain sum.
        total = xs[0]
        for x in xs[1:]:
            total = total + x
        return [total for _ in xs]


@register("cross_grid_sum_slice")
class CrossGridSumSlice(ExecLayer):
    """Sum across sub-grids, then each branch keeps its slice of the last dimension
    (include/lbann/layers/transform/cross_grid_sum_slice.hpp)."""
    max_parents = -1
    num_outputs = -1

    def setup(self, in_dims):
        k = len(in_dims)
        return [tuple(d[:-1]) + (d[-1] // k,) for d in in_dims]

    def forward(self, xs, training):
        total = xs[0]
        for x in xs[1:]:
            total = total + x
        k = len(xs)
        w = total.shape[-1] // k
        return [total[..., i * w:(i + 1) * w] for i in range(k)]
