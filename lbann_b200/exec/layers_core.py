"""Executable layers: io, learning, activations, losses, regularizers, operator layer.

Behaviour (shapes, defaults, weight names and initialisers, loss normalisation) follows the
reference layer by layer; the docstring of each class names the reference file.
"""
from __future__ import annotations

import math
from typing import List

import torch
import torch.nn.functional as F

from ..ops import native, nn
from ..ops import elementwise as ew
from ..proto import lbann_pb2 as pb
from .layer_base import ExecLayer, broadcast_list, prod, register, rows2d
from .weights import constant_default, he_normal_default

_FUSABLE_ACT = {"relu": (native.ACT_RELU, 0.0)}


# =============================================================================== io
@register("input")
class InputLayer(ExecLayer):
    """Pulls one data field of the current mini-batch (src/layers/io/input_layer.cpp:135-160)."""
    min_parents = max_parents = 0

    def setup(self, in_dims):
        field = self.params.data_field or "samples"
        self.field = field
        return [tuple(self.model.data_dims(field))]

    def forward(self, xs, training):
        x = self.model.current_inputs[self.field]
        return [self.cast_in(x)]


# =============================================================================== learning
@register("fully_connected")
class FullyConnected(ExecLayer):
    """y = W x + b on the flattened sample (src/layers/learning/fully_connected.cpp:119-247).
    Weights ``<name>_linearity_weights`` (He normal) and ``<name>_bias_weights`` (zero)."""

    def setup(self, in_dims):
        p = self.params
        self.in_size = prod(in_dims[0])
        out_dims = (int(p.num_neurons),)
        if self.hint_layer:
            out_dims = tuple(self.model.layer(self.hint_layer).out_dims[0])
        self.out_size = prod(out_dims)
        self.transpose = bool(p.transpose)
        shape = (self.in_size, self.out_size) if self.transpose else (self.out_size, self.in_size)
        self.w = self.get_weights(0, "linearity_weights", shape, he_normal_default,
                                  fan_in=self.in_size, fan_out=self.out_size)
        self.b = None
        if p.has_bias:
            self.b = self.get_weights(1, "bias_weights", (self.out_size,), constant_default(0.0))
        self.fused_act = (native.ACT_NONE, 0.0)
        return [out_dims]

    def forward(self, xs, training):
        x = rows2d(self.cast_in(xs[0]))
        par = self.model.parallel
        if par is not None and self.data_layout == "model_parallel" and par.tp_size > 1:
            y = par.tp_linear(self, x)
        elif sharded_linear_ok(self, par):
            y = self._sharded_forward(par, x)
        elif self.transpose:
            w = self.w.handle.master.to(x.dtype).t()
            y = F.linear(x, w, None if self.b is None else self.b.handle.master.to(x.dtype))
        else:
            y = nn.linear(x, self.w.handle, None if self.b is None else self.b.handle,
                          self.fused_act[0], self.fused_act[1])
        return [y.reshape(x.shape[0], *self.out_dims[0])]

    def _sharded_forward(self, par, x):
        return sharded_linear_forward(self, par, x)


def sharded_linear_forward(layer, par, x):
    """Weights flagged ``sharded``: every rank multiplies by its own block of output rows
    gathered tile by tile inside the GEMM (all-gather -> GEMM) and the weight gradient is
    reduce-scattered by the GEMM epilogue into the owner's rows (parallel/
    tensor_parallel.py::ShardedLinear).  The row block is a view of the arena's master
    copy, so optimizer and checkpoints see ordinary weights.  ``x``: [rows, in_size]."""
    from ..parallel.tensor_parallel import ShardedLinear
    P, r = par.world_size, par.comm.rank_in_trainer
    rows = layer.out_size // P
    lin = getattr(layer, "_sharded", None)
    if lin is None:
        lin = layer._sharded = ShardedLinear(par.group, layer.w.handle.master[r * rows:(r + 1) * rows])
    lin.w_shard = layer.w.handle.master[r * rows:(r + 1) * rows]
    y = lin(x)
    if layer.b is not None:
        y = y + layer.b.handle.master.to(y.dtype)
    if layer.fused_act[0] != native.ACT_NONE:
        from ..ops.gemm import _ACT_FN
        y = _ACT_FN[layer.fused_act[0]](y, layer.fused_act[1])
    return y


def sharded_linear_ok(layer, par) -> bool:
    return (par is not None and layer.w.sharded and par.world_size > 1 and not layer.transpose
            and layer.out_size % (128 * par.world_size) == 0 and layer.in_size % 8 == 0)


class _ConvBase(ExecLayer):
    supports_distconv = True
    supports_channel_parallel = True        # channel / filter partition (convolution only)

    def _common(self, in_dims):
        p = self.params
        nd = int(p.num_dims) or (len(in_dims[0]) - 1)
        self.nd = nd
        self.cin = int(in_dims[0][0])
        self.cout = int(p.out_channels)
        self.ksize = broadcast_list(p.kernel_size, nd, 1)
        self.stride = broadcast_list(p.stride, nd, 1)
        self.pad = broadcast_list(p.padding, nd, 0)
        self.dil = broadcast_list(p.dilation, nd, 1)
        self.groups = int(p.groups.value) if p.HasField("groups") else 1
        self.has_bias = bool(p.has_bias.value) if p.HasField("has_bias") else True
        self.fused_act = (native.ACT_NONE, 0.0)


@register("convolution")
class Convolution(_ConvBase):
    """N-d convolution, kernel ``<name>_kernel`` of shape K x C/groups x k... (He normal,
    fan-in = kernel volume * C/groups) and ``<name>_bias``
    (src/layers/learning/base_convolution.cpp:352-391, convolution.cpp)."""

    def setup(self, in_dims):
        self._common(in_dims)
        cg = self.cin // self.groups
        kvol = prod(self.ksize)
        self.w = self.get_weights(0, "kernel", (self.cout, cg) + self.ksize, he_normal_default,
                                  fan_in=kvol * cg, fan_out=kvol * self.cout // self.groups)
        self.b = self.get_weights(1, "bias", (self.cout,), constant_default(0.0)) if self.has_bias else None
        sp = in_dims[0][1:]
        out_sp = tuple((i + 2 * p - d * (k - 1) - 1) // s + 1
                       for i, p, d, k, s in zip(sp, self.pad, self.dil, self.ksize, self.stride))
        return [(self.cout,) + out_sp]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        dc = self.model.distconv
        pool = getattr(self, "fuse_pool_layer", None)
        fuse = None
        if pool is not None and (dc is None or dc.enabled(self) == dc.enabled(pool)):
            fuse = nn.PoolFusion()
        if dc is not None and dc.enabled(self):
            y = dc.convolution(self, x, fuse, pool)
        else:
            y = nn.convolution(x, self.w.handle, None if self.b is None else self.b.handle, self.ksize,
                               self.pad, self.stride, self.dil, self.groups, self.fused_act[0],
                               self.fused_act[1], getattr(self, "skip_act_grad", False), fuse)
        if pool is not None:
            pool.input_is_pooled = bool(fuse is not None and fuse.done)
        return [y]


@register("deconvolution")
class Deconvolution(_ConvBase):
    """Transposed convolution, kernel Cin x Cout/groups x k...
    (src/layers/learning/deconvolution.cpp)."""
    supports_channel_parallel = False

    def setup(self, in_dims):
        self._common(in_dims)
        p = self.params
        self.out_pad = broadcast_list(p.output_padding, self.nd, 0)
        cg = self.cout // self.groups
        kvol = prod(self.ksize)
        self.w = self.get_weights(0, "kernel", (self.cin, cg) + self.ksize, he_normal_default,
                                  fan_in=kvol * self.cin // self.groups, fan_out=kvol * cg)
        self.b = self.get_weights(1, "bias", (self.cout,), constant_default(0.0)) if self.has_bias else None
        sp = in_dims[0][1:]
        out_sp = tuple((i - 1) * s - 2 * p + d * (k - 1) + op + 1
                       for i, p, d, k, s, op in zip(sp, self.pad, self.dil, self.ksize, self.stride,
                                                    self.out_pad))
        return [(self.cout,) + out_sp]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        dc = self.model.distconv
        if dc is not None and dc.enabled(self):
            return [dc.deconvolution(self, x)]
        y = nn.deconvolution(x, self.w.handle, None if self.b is None else self.b.handle, self.ksize,
                             self.pad, self.stride, self.dil, self.out_pad, self.groups)
        return [y]


@register("channelwise_fully_connected")
class ChannelwiseFullyConnected(ExecLayer):
    supports_channel_parallel = True
    """The same fully-connected map applied to every channel (row) of the input
    (src/layers/learning/channelwise_fully_connected.cpp).  Weights ``<name>_matrix`` /
    ``<name>_bias`` in the front-end modules; default names ``_linearity_weights`` /
    ``_bias_weights`` here."""
    supports_distconv = True

    def setup(self, in_dims):
        p = self.params
        d = in_dims[0]
        self.channels = int(d[0])
        self.in_size = prod(d[1:])
        self.out_cdims = tuple(int(v) for v in p.output_channel_dims)
        self.out_size = prod(self.out_cdims)
        self.transpose = bool(p.transpose.value) if p.HasField("transpose") else False
        has_bias = bool(p.bias.value) if p.HasField("bias") else True
        shape = (self.in_size, self.out_size) if self.transpose else (self.out_size, self.in_size)
        self.w = self.get_weights(0, "linearity_weights", shape, he_normal_default,
                                  fan_in=self.in_size, fan_out=self.out_size)
        self.b = self.get_weights(1, "bias_weights", (self.out_size,), constant_default(0.0)) if has_bias else None
        self.fused_act = (native.ACT_NONE, 0.0)
        return [(self.channels,) + self.out_cdims]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        n = x.shape[0]
        dc = self.model.distconv
        c = self.channels
        if dc is not None and dc.channel_groups > 1 and dc.enabled(self):
            c //= dc.channel_groups                  # a channel partition holds a slice of the rows
        x2 = x.reshape(n, c, self.in_size)
        par = self.model.parallel
        if par is not None and self.data_layout == "model_parallel" and par.tp_size > 1:
            y = par.tp_linear(self, x2)
        elif sharded_linear_ok(self, par):
            # FSDP-style weights (``Weights(sharded=True)``): all-gather -> GEMM forward,
            # weight gradient reduce-scattered to the owners of the rows
            y = sharded_linear_forward(self, par, x2.reshape(-1, self.in_size)).reshape(
                n, c, self.out_size)
        elif self.transpose:
            w = self.w.handle.cast(x.dtype) if x.is_cuda else self.w.handle.master.to(x.dtype)
            if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16):
                y = _TransposedLinear.apply(x2, self.w.handle.master, self.w.handle)
            else:
                y = x2 @ w
            if self.b is not None:
                y = y + self.b.handle.master.to(y.dtype)
        else:
            y = nn.linear(x2, self.w.handle, None if self.b is None else self.b.handle,
                          self.fused_act[0], self.fused_act[1])
        return [y.reshape(n, c, *self.out_cdims)]


class _TransposedLinear(torch.autograd.Function):
    """y = x @ W for W stored [in, out] (tied embedding / LM head), native GEMMs both ways."""

    @staticmethod
    def forward(ctx, x, w_leaf, wh):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        w16 = wh.cast(x.dtype)
        ctx.save_for_backward(x2)
        ctx.meta = (wh, x.shape)
        from ..ops.gemm import gemm
        return gemm(x2, w16).reshape(*x.shape[:-1], w16.shape[1])

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm
        (x2,) = ctx.saved_tensors
        wh, xshape = ctx.meta
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = gemm(dy2, wh.cast(dy2.dtype), trans_b=True).reshape(xshape)
        if wh.grad is not None:
            gemm(x2, dy2, trans_a=True, out=wh.grad.view(wh.master.shape), beta=1.0)
            wh.mark_ready()
        return dx, None, None


@register("channelwise_scale_bias")
class ChannelwiseScaleBias(ExecLayer):
    """Per-channel affine map; one weights tensor [C, 2] = (scale, bias), init (1, 0)
    (src/layers/learning/channelwise_scale_bias.cpp)."""

    def setup(self, in_dims):
        c = int(in_dims[0][0])

        def init(shape, gen, fi, fo):
            t = torch.zeros(c, 2)
            t[:, 0] = 1.0
            return t.reshape(-1)
        self.w = self.get_weights(0, "weights", (c, 2), init)
        return [tuple(in_dims[0])]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        w = self.w.handle.master.to(x.dtype)
        shape = [1, -1] + [1] * (x.dim() - 2)
        return [x * w[:, 0].view(shape) + w[:, 1].view(shape)]


@register("entrywise_scale_bias")
class EntrywiseScaleBias(ExecLayer):
    """Per-entry affine map; weights [size, 2] (src/layers/learning/entrywise_scale_bias.cpp)."""

    def setup(self, in_dims):
        n = prod(in_dims[0])

        def init(shape, gen, fi, fo):
            t = torch.zeros(n, 2)
            t[:, 0] = 1.0
            return t.reshape(-1)
        self.w = self.get_weights(0, "weights", (n, 2), init)
        return [tuple(in_dims[0])]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        w = self.w.handle.master.to(x.dtype)
        d = self.in_dims[0]
        return [x * w[:, 0].view(1, *d) + w[:, 1].view(1, *d)]


@register("embedding")
class Embedding(ExecLayer):
    """Lookup table; weights ``<name>_weights`` hold one embedding vector per row
    (num_embeddings x embedding_dim, row-major: the same memory order as the reference's
    column-major embedding_dim x num_embeddings matrix, so value lists and checkpoints
    agree), out-of-range indices give zeros, ``padding_idx`` row gets no gradient
    (src/layers/learning/embedding.cpp, src/proto/layers.proto:1271-1276)."""

    def setup(self, in_dims):
        p = self.params
        self.num = int(p.num_embeddings)
        self.dim = int(p.embedding_dim)
        self.padding_idx = int(p.padding_idx.value) if p.HasField("padding_idx") else -1

        def init(shape, gen, fi, fo):
            return torch.randn(self.dim * self.num, generator=gen)
        self.w = self.get_weights(0, "weights", (self.num, self.dim), init)
        return [tuple(in_dims[0]) + (self.dim,)]

    def forward(self, xs, training):
        idx = xs[0].long()
        ok = (idx >= 0) & (idx < self.num)
        if self.padding_idx >= 0:
            ok = ok & (idx != self.padding_idx)
        dt = self.dtype or self.model.default_dtype
        table = self.w.handle.master
        out = F.embedding(idx.clamp(0, self.num - 1), table)
        out = out * ok.unsqueeze(-1).to(out.dtype)
        return [out.to(dt)]


@register("gru")
class GRU(ExecLayer):
    """Multi-layer GRU over a sequence input [seq, features] with an initial hidden state
    input [layers, hidden] (src/layers/learning/gru.cpp).  Weights per layer: ih_matrix,
    hh_matrix, ih_bias, hh_bias (gate order reset, update, new)."""
    min_parents = max_parents = 2

    def setup(self, in_dims):
        p = self.params
        self.hidden = int(p.hidden_size)
        self.layers = int(p.num_layers.value) if p.HasField("num_layers") else 1
        seq, feat = int(in_dims[0][0]), prod(in_dims[0][1:])
        self.seq, self.feat = seq, feat
        self.ws = []
        k = 1.0 / math.sqrt(self.hidden)

        def uinit(shape, gen, fi, fo):
            return (torch.rand(prod(shape), generator=gen) * 2 - 1) * k
        idx = 0
        for l in range(self.layers):
            isz = feat if l == 0 else self.hidden
            grp = []
            for suffix, shape in ((f"ih_matrix_l{l}", (3 * self.hidden, isz)),
                                  (f"hh_matrix_l{l}", (3 * self.hidden, self.hidden)),
                                  (f"ih_bias_l{l}", (3 * self.hidden,)),
                                  (f"hh_bias_l{l}", (3 * self.hidden,))):
                grp.append(self.get_weights(idx, suffix, shape, uinit))
                idx += 1
            self.ws.append(grp)
        return [(seq, self.hidden)]

    def forward(self, xs, training):
        x = self.cast_in(xs[0]).reshape(xs[0].shape[0], self.seq, self.feat)
        h0 = self.cast_in(xs[1]).reshape(xs[1].shape[0], self.layers, self.hidden)
        out = x
        for l, (wih, whh, bih, bhh) in enumerate(self.ws):
            wih, whh = wih.handle.master.to(x.dtype), whh.handle.master.to(x.dtype)
            bih, bhh = bih.handle.master.to(x.dtype), bhh.handle.master.to(x.dtype)
            h = h0[:, l]
            gi_all = F.linear(out, wih, bih)
            steps = []
            H = self.hidden
            # K-FAC (exec/kfac.py) needs, per stacked layer, the inputs of both products and
            # the error signals at their outputs: kept when it sets ``kfac_capture``
            cap = None
            if getattr(self, "kfac_capture", False) and gi_all.requires_grad:
                cap = {"x": out.detach(), "h_prev": [], "g_gi": None, "g_gh": [None] * self.seq}
                gi_all.register_hook(lambda g, c=cap: c.__setitem__("g_gi", g.detach()))
                if l == 0:
                    self.kfac_cache = []
                self.kfac_cache.append(cap)
            for t in range(self.seq):
                gi = gi_all[:, t]
                gh = F.linear(h, whh, bhh)
                if cap is not None:
                    cap["h_prev"].append(h.detach())
                    gh.register_hook(lambda g, c=cap, t=t: c["g_gh"].__setitem__(t, g.detach()))
                r = torch.sigmoid(gi[:, :H] + gh[:, :H])
                z = torch.sigmoid(gi[:, H:2 * H] + gh[:, H:2 * H])
                n = torch.tanh(gi[:, 2 * H:] + r * gh[:, 2 * H:])
                h = (1 - z) * n + z * h
                steps.append(h)
            out = torch.stack(steps, 1)
        return [out]


# =============================================================================== activations
class _Unary(ExecLayer):
    supports_channel_parallel = True
    op = "identity"
    supports_distconv = True

    def p0(self):
        return 0.0

    def forward(self, xs, training):
        if getattr(self, "fused_into_parent", False):
            return [xs[0]]
        return [ew.unary(self.op, self.cast_in(xs[0]), self.p0(), 0.0)]


@register("relu")
class Relu(_Unary):
    """src/layers/activations/relu.cu"""
    op = "relu"


@register("leaky_relu")
class LeakyRelu(_Unary):
    """negative_slope defaults to 0.01 (src/layers/activations/leaky_relu.cu)."""
    op = "leaky_relu"

    def p0(self):
        return float(self.params.negative_slope) or 0.01


@register("elu")
class Elu(_Unary):
    """alpha defaults to 1 (src/layers/activations/elu.cu)."""
    op = "elu"

    def p0(self):
        return float(self.params.alpha) or 1.0


@register("identity")
class Identity(ExecLayer):
    supports_channel_parallel = True
    supports_distconv = True

    def forward(self, xs, training):
        return [xs[0]]


@register("softmax")
class Softmax(ExecLayer):
    """Softmax over the whole sample ("instance") or over channels for every spatial
    position ("channel") (src/layers/activations/softmax.cu:70-240)."""
    supports_distconv = True
    log = False

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        if getattr(self, "fused_into_child", False):
            return [x]          # the cross-entropy child consumes the logits
        mode = (self.params.softmax_mode or "instance") if hasattr(self.params, "softmax_mode") else "instance"
        if mode == "channel" and x.dim() > 2:
            xm = x.movedim(1, -1)
            y = nn.softmax_lastdim(xm.contiguous(), self.log)
            return [y.movedim(-1, 1)]
        n = x.shape[0]
        par = self.model.parallel
        if par is not None and self.data_layout == "model_parallel" and par.tp_size > 1:
            return [par.tp_softmax(rows2d(x), self.log).reshape(x.shape)]
        return [nn.softmax_lastdim(rows2d(x), self.log).reshape(x.shape)]


@register("log_softmax")
class LogSoftmax(Softmax):
    """src/layers/activations/log_softmax.cu"""
    log = True


# =============================================================================== losses
class _SampleLoss(ExecLayer):
    min_parents = max_parents = 2
    kind = "mean_squared_error"
    supports_distconv = True

    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        a = self.cast_in(xs[0])
        b = self.cast_in(xs[1]).to(a.dtype)
        dc = self.model.distconv
        if dc is not None and dc.enabled(self):
            return [dc.sample_loss(self, self.kind, a, b)]
        return [nn.sample_loss(self.kind, a, b.reshape(a.shape)).reshape(-1, 1)]


@register("mean_squared_error")
class MeanSquaredError(_SampleLoss):
    """Mean over the sample's entries of (a-b)^2 (src/layers/loss/mean_squared_error.cu:74)."""
    kind = "mean_squared_error"


@register("mean_absolute_error")
class MeanAbsoluteError(_SampleLoss):
    """src/layers/loss/mean_absolute_error.cu"""
    kind = "mean_absolute_error"


@register("cross_entropy")
class CrossEntropy(ExecLayer):
    """-sum y log(yhat) over entries with y > 0; with ``use_labels`` the second input holds
    integer class ids per spatial position and the first is [classes, positions...]
    (src/layers/loss/cross_entropy.cu:55-73, cross_entropy_impl.hpp)."""
    min_parents = max_parents = 2
    supports_distconv = True

    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        p = self.cast_in(xs[0])
        n = p.shape[0]
        dc = self.model.distconv
        if dc is not None and dc.enabled(self):
            return [dc.cross_entropy(self, p, xs[1])]
        fused = getattr(self, "fused_logits", None)
        if self.params.use_labels:
            C = p.shape[1]
            lab = rows2d(xs[1]).long()
            pm = p.reshape(n, C, -1).movedim(1, -1)            # n, positions, C
            if fused is not None:
                loss = nn.softmax_cross_entropy(pm.contiguous(), lab)
            else:
                ok = (lab >= 0) & (lab < C)
                picked = pm.float().gather(2, lab.clamp(0, C - 1).unsqueeze(-1)).squeeze(-1)
                loss = torch.where(ok, -torch.log(picked), torch.zeros_like(picked))
            return [loss.sum(1, keepdim=True)]
        t = self.cast_in(xs[1]).to(p.dtype).reshape(p.shape)
        if fused is not None:
            # parent softmax was folded away: p holds logits
            lp = nn.softmax_lastdim(rows2d(p), log=True)
            return [-(rows2d(t).float() * lp.float()).sum(1, keepdim=True)]
        return [nn.sample_loss("cross_entropy", p, t).reshape(-1, 1)]


@register("categorical_accuracy")
class CategoricalAccuracy(ExecLayer):
    """1 if argmax(prediction) == argmax(label) (src/layers/loss/categorical_accuracy.cu)."""
    min_parents = max_parents = 2
    k = 1

    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        n = xs[0].shape[0]
        with torch.no_grad():
            pred = rows2d(xs[0])
            lab = rows2d(xs[1])
            if lab.shape[1] == pred.shape[1]:
                lab = lab.argmax(1)
            else:
                lab = lab[:, 0].long()
            return [nn.topk_accuracy(pred, lab, self.k).reshape(n, 1)]


@register("top_k_categorical_accuracy")
class TopKCategoricalAccuracy(CategoricalAccuracy):
    """src/layers/loss/top_k_categorical_accuracy.cu"""

    def setup(self, in_dims):
        self.k = int(self.params.k) or 1
        return [(1,)]


@register("l1_norm")
class L1Norm(ExecLayer):
    """src/layers/loss/l1_norm.cu"""
    kind = "l1_norm"

    def setup(self, in_dims):
        return [(1,)]

    def forward(self, xs, training):
        return [nn.sample_loss(self.kind, self.cast_in(xs[0])).reshape(-1, 1)]


@register("l2_norm2")
class L2Norm2(L1Norm):
    """src/layers/loss/l2_norm2.cu"""
    kind = "l2_norm2"


# =============================================================================== regularizers
@register("batch_normalization")
class BatchNormalization(ExecLayer):
    """Per-channel batch norm.  ``statistics_group_size``: < 0 global, 0/1 local, k > 1
    groups of k ranks; decay 0.9, epsilon 1e-5, Bessel-corrected variance clamped at
    epsilon; weights scale, bias, running_mean, running_variance
    (src/layers/regularizers/batch_normalization.cu:139-153,393-403,
    batch_normalization_builder.cpp:48-76)."""
    supports_distconv = True

    def setup(self, in_dims):
        p = self.params
        c = int(in_dims[0][0])
        self.decay = float(p.decay) or 0.9
        self.eps = float(p.epsilon) or 1e-5
        g = int(p.statistics_group_size)
        self.stats_group = 0 if g < 0 else (1 if g == 0 else g)
        self.bessel = not bool(p.no_bessel_correction)
        self.scale = self.get_weights(0, "scale", (c,), constant_default(float(p.scale_init) or 1.0))
        self.bias = self.get_weights(1, "bias", (c,), constant_default(float(p.bias_init)))
        self.run_mean = self.get_weights(2, "running_mean", (c,), constant_default(0.0), optimizer=False)
        self.run_var = self.get_weights(3, "running_variance", (c,), constant_default(1.0), optimizer=False)
        self.fused_act = (native.ACT_NONE, 0.0)
        return [tuple(in_dims[0])]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        reduce_fn, count_scale = None, 1.0
        par = self.model.parallel
        dc = self.model.distconv
        if dc is not None and dc.enabled(self):
            reduce_fn, count_scale = dc.bn_reduction(self)
        elif par is not None and self.stats_group != 1 and par.dp_size > 1:
            reduce_fn, count_scale = par.bn_reduction(self.stats_group)
        if reduce_fn is not None and training:
            count_scale = self.exact_count_scale(x, count_scale)
        squeeze = False
        if x.dim() == 2:
            x = x.unsqueeze(-1)
            squeeze = True
        y = nn.batch_norm(x, self.scale.handle, self.bias.handle,
                          self.run_mean.handle.master.detach(), self.run_var.handle.master.detach(),
                          training, self.eps, self.decay, self.bessel, reduce_fn, count_scale,
                          self.fused_act[0], self.fused_act[1])
        return [y.squeeze(-1) if squeeze else y]


    def exact_count_scale(self, x, count_scale: float) -> float:
        """Statistics over the whole trainer: entries per channel of the whole mini-batch divided
        by this rank's, which is the number of ranks only while every rank holds the same share
        (the last mini-batch of an epoch, or a sample-parallel stretch behind a partitioned one,
        may deal 2 + 1 samples).  The reference counts the global mini-batch the same way
        (src/layers/regularizers/batch_normalization.cu:139-153)."""
        m, par = self.model, self.model.parallel
        if (par is None or count_scale != float(par.world_size) or par.tp_size != 1
                or getattr(m, "subgrid", None) is not None or not getattr(m, "_global_mb_given", False)):
            return count_scale
        local = x.numel() // max(int(x.shape[1]), 1)
        total = int(m._global_mb) * prod(self.in_dims[0][1:])
        return total / local if local > 0 else count_scale


@register("entrywise_batch_normalization")
class EntrywiseBatchNormalization(ExecLayer):
    """Statistics per entry over the mini-batch (src/layers/regularizers/
    entrywise_batch_normalization.cu); weights running_mean, running_variance."""

    def setup(self, in_dims):
        p = self.params
        n = prod(in_dims[0])
        self.decay = float(p.decay) or 0.9
        self.eps = float(p.epsilon) or 1e-5
        self.run_mean = self.get_weights(0, "running_mean", (n,), constant_default(0.0), optimizer=False)
        self.run_var = self.get_weights(1, "running_variance", (n,), constant_default(1.0), optimizer=False)
        return [tuple(in_dims[0])]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        n = x.shape[0]
        xf = rows2d(x).float()
        rm, rv = self.run_mean.handle.master.detach(), self.run_var.handle.master.detach()
        if training:
            par = self.model.parallel
            s = torch.stack([xf.sum(0), (xf * xf).sum(0)])
            cnt = float(n)
            if par is not None and par.dp_size > 1:
                s = nn._ReduceSum.apply(s, par.allreduce_sum_inplace)
                cnt *= par.dp_size
            mean = s[0] / cnt
            var = torch.clamp(s[1] / cnt - mean * mean, min=0.0)
            with torch.no_grad():
                unbiased = var * (cnt / max(cnt - 1.0, 1.0))
                rm.mul_(self.decay).add_((1 - self.decay) * mean.detach())
                rv.mul_(self.decay).add_((1 - self.decay) * unbiased.detach())
        else:
            mean, var = rm, rv
        y = (xf - mean) * torch.rsqrt(var + self.eps)
        return [y.reshape(x.shape).to(x.dtype)]


@register("layer_norm")
class LayerNorm(ExecLayer):
    """Normalise each sample over dims [start_dim:], optional scale/bias weights
    ``<name>_scale`` (1) / ``<name>_bias`` (0); epsilon 1e-5
    (src/layers/regularizers/layer_norm.cu, src/proto/layers.proto:574-603)."""

    def setup(self, in_dims):
        p = self.params
        d = in_dims[0]
        self.eps = float(p.epsilon.value) if p.HasField("epsilon") else 1e-5
        sd = int(p.start_dim)
        if sd < 0:
            sd += len(d)
        self.norm_dims = tuple(d[sd:])
        self.norm_size = prod(self.norm_dims)
        self.scale = self.get_weights(0, "scale", self.norm_dims, constant_default(1.0)) if p.scale else None
        self.bias = self.get_weights(1 if p.scale else 0, "bias", self.norm_dims,
                                     constant_default(0.0)) if p.bias else None
        return [tuple(d)]

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        y = nn.layer_norm(x, self.norm_size, self.scale.handle if self.scale else None,
                          self.bias.handle if self.bias else None, self.eps)
        return [y]


@register("instance_norm")
class InstanceNorm(ExecLayer):
    """Per-sample, per-channel normalisation (src/layers/regularizers/instance_norm.cu)."""

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        eps = float(self.params.epsilon.value) if self.params.HasField("epsilon") else 1e-5
        n, c = x.shape[0], x.shape[1]
        y = nn.layer_norm(x.reshape(n * c, -1), prod(x.shape[2:]), None, None, eps)
        return [y.reshape(x.shape)]


@register("dropout")
class Dropout(ExecLayer):
    supports_channel_parallel = True
    """Inverted dropout with keep probability ``keep_prob`` (default 0.5)
    (src/layers/regularizers/dropout.cpp)."""

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        keep = float(self.params.keep_prob) or 0.5
        keep = getattr(self, "keep_prob_override", keep)
        if not training or keep >= 1.0:
            return [x]
        return [F.dropout(x, 1.0 - keep, True)]


@register("selu_dropout")
class SeluDropout(ExecLayer):
    """Alpha dropout for SELU networks (src/layers/regularizers/selu_dropout.cpp)."""

    def forward(self, xs, training):
        x = self.cast_in(xs[0])
        p = self.params
        keep = float(p.keep_prob) or 0.95
        if not training:
            return [x]
        alpha = float(p.alpha) or 1.6732632423543772
        scale = float(p.scale) or 1.0507009873554805
        ap = -scale * alpha
        a = (keep + ap * ap * keep * (1 - keep)) ** -0.5
        b = -a * ap * (1 - keep)
        mask = (torch.rand_like(x, dtype=torch.float32) < keep).to(x.dtype)
        return [a * (x * mask + ap * (1 - mask)) + b]


@register("local_response_normalization")
class LocalResponseNormalization(ExecLayer):
    """Cross-channel LRN (include/lbann/layers/regularizers/local_response_normalization.hpp)."""

    def forward(self, xs, training):
        p = self.params
        x = self.cast_in(xs[0])
        return [F.local_response_norm(x.float(), int(p.window_width) or 5, float(p.lrn_alpha) or 1e-4,
                                      float(p.lrn_beta) or 0.75, float(p.lrn_k) or 1.0).to(x.dtype)]


# =============================================================================== operator layer
def _snake(name: str) -> str:
    out = []
    for i, ch in enumerate(name):
        if ch.isupper() and i and (not name[i - 1].isupper() or (i + 1 < len(name) and name[i + 1].islower())):
            out.append("_")
        out.append(ch.lower())
    return "".join(out)




@register("operator_layer")
class OperatorLayer(ExecLayer):
    supports_channel_parallel = True
    """A chain of entrywise operators (include/lbann/layers/operator_layer_impl.hpp,
    src/proto/operators.proto).  A single operator is the common case."""
    max_parents = -1
    supports_distconv = True

    def setup(self, in_dims):
        self.ops = []
        for op in self.params.ops:
            type_name = op.parameters.type_url.split(".")[-1]       # e.g. ScaleOperator
            msg = getattr(pb, type_name)()
            op.parameters.Unpack(msg)
            short = _snake(type_name[:-len("Operator")])
            short = {"erf_inv": "erfinv"}.get(short, short)
            self.ops.append((short, msg))
        return [tuple(in_dims[0])]

    def forward(self, xs, training):
        if getattr(self, "fused_into_child", False):
            return [self.cast_in(xs[0])]      # the consumer applies this operator itself
        xs = [self.cast_in(x) for x in xs]
        cur = xs
        for short, msg in self.ops:
            cur = [self._apply(short, msg, cur)]
        return cur

    def _apply(self, short, msg, xs):
        if short in ew.BINARY_CODE:
            a, b = xs[0], xs[1]
            if b.shape != a.shape:
                if b.numel() == a.numel():
                    b = b.reshape(a.shape)
                else:
                    # operands with unit dims (a mask shared by all heads, a per-row scale):
                    # broadcast instead of asking the graph to tessellate them
                    if a.numel() < b.numel():
                        a = a.expand(torch.broadcast_shapes(a.shape, b.shape))
                    else:
                        b = b.expand(torch.broadcast_shapes(a.shape, b.shape))
                    a, b = a.contiguous(), b.to(a.dtype).contiguous()
            if (short == "add" and len(self.ops) == 1
                    and getattr(self, "fused_act", (native.ACT_NONE, 0.0))[0] == native.ACT_RELU):
                return ew.add_relu(a, b.to(a.dtype))      # the ReLU that follows is folded in
            return ew.binary(short, a, b.to(a.dtype))
        if short == "clamp":
            return ew.unary("clamp", xs[0], float(msg.min), float(msg.max))
        if short == "select":
            return self._select(msg, xs)
        if short == "log_softmax":
            n = xs[0].shape[0]
            return nn.softmax_lastdim(rows2d(xs[0]), True).reshape(xs[0].shape)
        if short in ew.UNARY_CODE:
            c = float(getattr(msg, "constant", 0.0)) if hasattr(msg, "constant") else 0.0
            return ew.unary(short, xs[0], c, 0.0)
        raise NotImplementedError(f"operator {short}")

    @staticmethod
    def _select(msg, xs):
        pred = xs[0]
        eps = float(msg.epsilon)
        cond = (pred - float(msg.value)).abs() <= eps
        t = xs[1] if not msg.constant_if_true else torch.full_like(pred, float(msg.value_if_true))
        rest = xs[2:] if not msg.constant_if_true else xs[1:]
        f = rest[0] if not msg.constant_if_false else torch.full_like(pred, float(msg.value_if_false))
        return torch.where(cond, t, f)
