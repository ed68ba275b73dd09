"""Executable model: layer graph + weights arena + objective + metrics.

Mirrors the responsibilities of the reference's ``model`` class (src/models/model.cpp):
set-up order (topology check -> execution order -> layer set-up -> weights sorted by name
-> objective / metrics), forward / backward / update, per-mode statistics.  Differences by
design: backward is PyTorch autograd over the layers' forward functions; all weights live
in one flat arena updated by a single fused optimizer launch; split / dummy / evaluation
helper layers are implicit (a tensor may simply feed several children).
"""
from __future__ import annotations

import os
import time
from collections import OrderedDict, defaultdict
from typing import Callable, Dict, List, Optional

import torch

from ..ops import native
from ..ops.optim import ParameterArena
from ..proto import lbann_pb2 as pb
from . import layers_core, layers_misc  # noqa: F401  (populate the registry)
from .layer_base import LAYER_REGISTRY, ExecLayer
from .weights import ExecWeights, optimizer_from_proto

MODES = ("training", "validation", "testing", "prediction", "tournament")


class LbannError(RuntimeError):
    pass


class ModeStats:
    """Running sums for one execution mode, kept on the device (no per-step host sync)."""

    def __init__(self, device, num_metrics):
        self.obj_sum = torch.zeros((), dtype=torch.float64, device=device)
        self.samples = 0
        self.metric_sums = [torch.zeros((), dtype=torch.float64, device=device)
                            for _ in range(num_metrics)]

    def reset(self):
        self.obj_sum.zero_()
        self.samples = 0
        for m in self.metric_sums:
            m.zero_()


class ExecMetric:
    def __init__(self, name, layer_name, unit=""):
        self.name, self.layer_name, self.unit = name, layer_name, unit


class ExecModel:
    def __init__(self, model_pb, default_optimizer_pb=None, *, device="cpu",
                 default_dtype=torch.float32, data_dims: Optional[Callable] = None,
                 slice_points: Optional[Callable] = None, comm=None, parallel=None,
                 distconv=None, seed: int = 0, arena_allocator=None):
        self.proto = model_pb
        self.name = model_pb.name or "model"
        self.device = torch.device(device)
        self.default_dtype = default_dtype
        self._data_dims = data_dims or (lambda field: (1,))
        self._slice_points = slice_points
        self.comm = comm
        self.parallel = parallel
        self.distconv = distconv
        self.seed = int(seed)
        self.default_optimizer = optimizer_from_proto(default_optimizer_pb) \
            if default_optimizer_pb is not None else (None, {})
        if self.default_optimizer[0] is None:
            self.default_optimizer = ("none", {})
        self.layers: List[ExecLayer] = []
        self.layers_by_name: Dict[str, ExecLayer] = {}
        self.weights: List[ExecWeights] = []
        self.weights_by_name: Dict[str, ExecWeights] = {}
        self.arena: Optional[ParameterArena] = None
        self.arena_allocator = arena_allocator
        self.callbacks = []
        self.metrics: List[ExecMetric] = []
        self.objective_terms = []      # (layer_name, scale)
        self.l2_terms = []             # (scale, [weights names])
        self.acts: Dict[str, List[torch.Tensor]] = {}
        self.current_inputs: Dict[str, torch.Tensor] = {}
        self.current_mini_batch_size = 0
        self._global_mb = 0
        self._mb_offset = 0
        self.stats: Dict[str, ModeStats] = {}
        self.last_objective = None
        self.num_epochs = int(model_pb.num_epochs)
        self.amp_enabled = bool(model_pb.amp.enabled) if model_pb.HasField("amp") else False
        amp = model_pb.amp
        self._amp_scale_host = float(amp.init_scale) or 65536.0
        self._amp_state = None      # CUDA: [scale, 1 / scale, clean steps, skipped steps] on the device
        self.amp_growth = float(amp.growth_factor) or 2.0
        self.amp_backoff = float(amp.backoff_factor) or 0.5
        self.amp_interval = int(amp.growth_interval) or 2000
        self._amp_good_steps = 0
        self._amp_skipped = 0
        self._gen = None
        self.sync_layers = False       # debugging: synchronise after every layer
        self._graph_mode = None        # decided at the first training step
        self._graphs = {}
        self.layer_timing = False
        self.is_setup = False

    # ------------------------------------------------------------------ helpers used by layers
    def data_dims(self, field):
        return tuple(int(d) for d in self._data_dims(field))

    def slice_points_from_reader(self, which):
        if self._slice_points is None:
            raise LbannError("no data reader provides slice points")
        return self._slice_points(which)

    def layer(self, name) -> ExecLayer:
        return self.layers_by_name[name]

    def activation(self, layer_name, index=0) -> torch.Tensor:
        return self.acts[layer_name][index]

    def add_weights(self, w: ExecWeights):
        if w.name in self.weights_by_name:
            raise LbannError(f"duplicate weights name '{w.name}'")
        self.weights.append(w)
        self.weights_by_name[w.name] = w

    def generator(self):
        if self._gen is None or self._gen.device != self.device:
            self._gen = torch.Generator(device=self.device)
            rank = self.comm.rank_in_world if self.comm is not None else 0
            self._gen.manual_seed(self.seed * 7919 + 17 * rank + 1)
        return self._gen

    def global_mini_batch_size(self):
        return self._global_mb

    def mini_batch_offset(self):
        return self._mb_offset

    # ------------------------------------------------------------------ set-up
    def setup(self):
        m = self.proto
        for wp in m.weights:
            self.add_weights(ExecWeights(wp.name, wp))
        seen = set()
        for lp in m.layer:
            if not lp.name:
                raise LbannError("layer without a name")
            if lp.name in seen:
                raise LbannError(f"duplicate layer name '{lp.name}'")
            seen.add(lp.name)
            t = lp.WhichOneof("layer_type")
            if t not in LAYER_REGISTRY:
                raise LbannError(f"layer '{lp.name}': unsupported layer type '{t}'")
            layer = LAYER_REGISTRY[t](lp, self)
            self.layers.append(layer)
            self.layers_by_name[layer.name] = layer
        self._setup_topology()
        self._setup_execution_order()
        if self.parallel is not None:
            self.parallel.prepare_model(self)
        self.subgrid = getattr(self.parallel, "subgrid", None) if self.parallel is not None else None
        if self.subgrid is not None:
            self.subgrid.resolve_tags(self)
        else:
            for l in self.layers:
                l.grid_tag = 0
        if self.distconv is not None:
            self.distconv.prepare_model(self)
        for layer in self.layers:
            in_dims = []
            for pn in layer.parent_names:
                parent = self.layers_by_name[pn]
                in_dims.append(parent.out_dims[self._slot(parent, layer)])
            layer.in_dims = [tuple(d) for d in in_dims]
            for wn in layer.weight_names:
                if wn and wn not in self.weights_by_name:
                    raise LbannError(f"layer '{layer.name}' refers to unknown weights '{wn}'")
            layer.out_dims = [tuple(int(x) for x in d) for d in layer.setup(layer.in_dims)]
        self._setup_weights()
        self._setup_objective()
        self._fuse_activations()
        self._fuse_softmax_cross_entropy()
        self._fuse_attention_scores()
        self._fuse_attention()
        for mode in MODES:
            self.stats[mode] = ModeStats(self.device, len(self.metrics))
        # LBANN_PHASE_TIMING=1: CUDA events between the phases of a step launched from the host;
        # LBANN_PHASE_TIMING=graph: the step is replayed as THREE graphs (forward / backward +
        # gradient reduction / update) with events between them, i.e. the phase times of the
        # graph-launched step, free of host launch gaps
        pt_mode = os.environ.get("LBANN_PHASE_TIMING")
        self._phase_timer = ExecModel._PhaseTimer(self.device) if pt_mode else None
        self._phase_graphs = pt_mode == "graph"
        self.is_setup = True
        return self

    def _setup_topology(self):
        by = self.layers_by_name
        for l in self.layers:
            for pn in l.parent_names:
                if pn not in by:
                    raise LbannError(f"layer '{l.name}' has unknown parent '{pn}'")
            for cn in l.child_names:
                if cn not in by:
                    raise LbannError(f"layer '{l.name}' has unknown child '{cn}'")
        # reciprocate edges: a parent listed by the child must list the child and vice versa
        for l in self.layers:
            for pn in l.parent_names:
                p = by[pn]
                if p.child_names.count(l.name) < l.parent_names.count(pn):
                    p.child_names.append(l.name)
            for cn in l.child_names:
                c = by[cn]
                if c.parent_names.count(l.name) < l.child_names.count(cn):
                    c.parent_names.append(l.name)
        for l in self.layers:
            l.parents = [by[n] for n in l.parent_names]
            l.children = [by[n] for n in l.child_names]
            n = len(l.parents)
            if n < l.min_parents or (l.max_parents >= 0 and n > l.max_parents):
                raise LbannError(f"layer '{l.name}' ({l.type}) has {n} parents")

    def _setup_execution_order(self):
        indeg = {l.name: len(l.parent_names) for l in self.layers}
        order, ready = [], [l for l in self.layers if indeg[l.name] == 0]
        ready.sort(key=lambda l: 0 if l.type == "input" else 1)   # inputs first
        pos = {l.name: i for i, l in enumerate(self.layers)}
        while ready:
            l = ready.pop(0)
            order.append(l)
            nxt = []
            for c in l.children:
                indeg[c.name] -= 1
                if indeg[c.name] == 0:
                    nxt.append(c)
            ready.extend(sorted(set(nxt), key=lambda x: pos[x.name]))
        if len(order) != len(self.layers):
            raise LbannError("layer graph has a cycle")
        self.layers = order

    @staticmethod
    def _slot(parent: ExecLayer, child: ExecLayer, occurrence: int = 0) -> int:
        if parent.num_outputs == 1:
            return 0
        idxs = [i for i, n in enumerate(parent.child_names) if n == child.name]
        return idxs[min(occurrence, len(idxs) - 1)]

    def _setup_weights(self):
        # deterministic order: sorted by name (src/models/model.cpp:1138-1153)
        self.weights.sort(key=lambda w: w.name)
        compute = self.default_dtype if (self.device.type == "cuda" and self.default_dtype in
                                         (torch.float16, torch.bfloat16)) else None
        self.arena = ParameterArena(self.device, compute_dtype=compute,
                                    allocator=self.arena_allocator)
        used = [w for w in self.weights if w.shape is not None]
        for w in used:
            w.bind(self.arena)
        self.arena.materialise()
        for w in used:
            w.materialise(self.default_optimizer, self.seed)
        self.weights = used
        self.weights_by_name = {w.name: w for w in used}
        if self.parallel is not None:
            self.parallel.sync_initial_weights(self)
        self.arena.refresh_compute()

    def _setup_objective(self):
        obj = self.proto.objective_function
        for t in obj.layer_term:
            if t.layer not in self.layers_by_name:
                raise LbannError(f"objective refers to unknown layer '{t.layer}'")
            self.objective_terms.append((t.layer, float(t.scale_factor) if t.scale_factor else 1.0))
        for t in obj.l2_weight_regularization:
            names = [n for s in t.weights for n in s.split()] or [w.name for w in self.weights]
            scale = float(t.scale_factor) if t.scale_factor else 1.0
            self.l2_terms.append((scale, names))
            for n in names:
                w = self.weights_by_name.get(n)
                if w is not None and w.has_optimizer():
                    w.slot.l2 += scale
        for mp in self.proto.metric:
            which = mp.WhichOneof("metric_type")
            if which == "layer_metric":
                lm = mp.layer_metric
                if lm.layer not in self.layers_by_name:
                    raise LbannError(f"metric refers to unknown layer '{lm.layer}'")
                self.metrics.append(ExecMetric(lm.name or lm.layer, lm.layer, lm.unit))
            elif which is not None:
                from .metrics import make_external_metric
                self.metrics.append(make_external_metric(which, getattr(mp, which)))

    def _fuse_activations(self):
        """Fold ReLU / leaky ReLU that directly follows a convolution, fully-connected or
        batch-norm layer into that layer's kernel epilogue (CUDA 16-bit path only)."""
        if self.device.type != "cuda" or self.default_dtype not in (torch.float16, torch.bfloat16):
            return
        protected = {n for n, _ in self.objective_terms} | {m.layer_name for m in self.metrics
                                                            if getattr(m, "layer_name", None)}
        for l in self.layers:
            if l.type not in ("convolution", "fully_connected", "batch_normalization",
                              "channelwise_fully_connected", "sum", "operator_layer"):
                continue
            if l.type == "operator_layer" and [o for o, _ in getattr(l, "ops", [])] != ["add"]:
                continue
            if len(l.children) != 1 or l.name in protected:
                continue
            c = l.children[0]
            if l.type in ("sum", "operator_layer") and (c.type != "relu" or len(l.parent_names) < 2):
                continue          # residual addition: only a plain ReLU is folded in
            if c.type == "relu":
                act = (native.ACT_RELU, 0.0)
            elif c.type == "leaky_relu":
                act = (native.ACT_LEAKY, c.p0())
            else:
                continue
            if (l.dtype or self.default_dtype) != (c.dtype or self.default_dtype):
                continue
            if getattr(l, "transpose", False) or getattr(l, "groups", 1) != 1:
                continue
            if l.data_layout == "model_parallel":
                continue
            if (l.type == "convolution" and self.distconv is not None and self.distconv.channel_groups > 1
                    and self.distconv.enabled(l)):
                continue          # channel / filter partition: the general path, nothing folded in
            l.fused_act = act
            c.fused_into_parent = True
            # conv -> (fused act) -> max pooling: the pooling backward kernel also applies the
            # activation gradient, so the convolution's backward skips that pass
            if (l.type == "convolution" and len(c.children) == 1 and c.name not in protected
                    and c.children[0].type == "pooling" and c.children[0].mode == "max"
                    and l.cout % 8 == 0):
                pool = c.children[0]
                pool.bwd_act = act
                l.skip_act_grad = True
                # a first-layer convolution (<= 4 channels, 3^3 filter) followed by 2^3 / stride-2
                # max pooling runs both in one kernel where the shapes allow (ops/nn.py)
                hinted = {getattr(x, "hint_layer", None) for x in self.layers}
                if (l.nd == 3 and l.cin <= 4 and tuple(l.ksize) == (3, 3, 3)
                        and tuple(l.stride) == (1, 1, 1) and tuple(l.dil) == (1, 1, 1)
                        and tuple(pool.k) == (2, 2, 2) and tuple(pool.stride) == (2, 2, 2)
                        and tuple(pool.pad) == (0, 0, 0) and pool.name not in protected
                        and pool.name not in hinted):
                    l.fuse_pool_layer = pool

    def _fuse_softmax_cross_entropy(self):
        """softmax over channels -> cross-entropy with integer labels: the softmax layer
        passes its input through and the loss layer runs the fused softmax-cross-entropy
        kernel on the logits (one pass, no probability tensor)."""
        protected = {n for n, _ in self.objective_terms} | {m.layer_name for m in self.metrics
                                                            if getattr(m, "layer_name", None)}
        for l in self.layers:
            if l.type != "cross_entropy" or not l.params.use_labels or not l.parents:
                continue
            sm = l.parents[0]
            if sm.type != "softmax" or len(sm.children) != 1 or sm.name in protected:
                continue
            mode = (getattr(sm.params, "softmax_mode", "") or "instance")
            if mode != "channel" or len(sm.in_dims[0]) < 2:
                continue
            if self.distconv is not None and self.distconv.enabled(l):
                continue
            sm.fused_into_child = True
            l.fused_logits = True

    def _fuse_attention_scores(self):
        """QK^T -> scale -> (+ causal mask) -> softmax: fold the scaling and the causal mask
        into the softmax kernel, which then reads the raw scores once instead of three
        element-wise passes over the [heads, S, S] tensor.  A mask qualifies when it is a
        constant (optimizer-less) weights layer holding 0 on and below the diagonal and a
        large negative number above it."""
        if self.distconv is not None and getattr(self.distconv, "channel_groups", 1) > 1:
            return          # the attention chain is partitioned over tokens: keep its layers apart
        forced = os.environ.get("LBANN_FORCE_ATTENTION_FUSION")     # CPU tests of the graph rewrite
        if (self.device.type != "cuda" and not forced) or os.environ.get("LBANN_DISABLE_ATTENTION_FUSION"):
            return
        protected = {n for n, _ in self.objective_terms} | {m.layer_name for m in self.metrics
                                                            if getattr(m, "layer_name", None)}

        def single_op(l, short):
            return (l.type == "operator_layer" and len(getattr(l, "ops", [])) == 1
                    and l.ops[0][0] == short and len(l.children) == 1 and l.name not in protected)

        for sm in self.layers:
            if sm.type != "channelwise_softmax" or not sm.parents:
                continue
            nd = len(sm.in_dims[0])
            dim = int(sm.params.dim)
            if not sm.params.single_dim_mode or (dim + nd) % nd != nd - 1 or nd < 2:
                continue
            S = sm.in_dims[0][-1]
            cur = sm.parents[0]
            mask_layer = None
            if single_op(cur, "add") and len(cur.parents) == 2 and cur.parents[1].type == "weights_layer":
                wl = cur.parents[1]
                w = wl.w.handle.master.detach().float().reshape(-1, S, S) if wl.out_dims[0][-2:] == (S, S) \
                    and sm.in_dims[0][-2] == S else None
                if w is not None and not wl.w.has_optimizer():
                    tri = torch.triu(torch.ones(S, S, dtype=torch.bool, device=w.device), 1)
                    if bool((w[:, ~tri] == 0).all()) and bool((w[:, tri] <= -1e4).all()):
                        mask_layer = cur
                        cur = cur.parents[0]
            scale = None
            if single_op(cur, "scale"):
                scale = float(cur.ops[0][1].constant)
            if mask_layer is None and scale is None:
                continue
            if mask_layer is not None:
                mask_layer.fused_into_child = True
                sm.fused_causal = S
            if scale is not None:
                cur.fused_into_child = True
                sm.fused_scale = scale

    def _fuse_attention(self):
        """The whole scaled-dot-product sub-graph that the front end emits for batched heads
        (python/lbann/modules/transformer/attention.py:215-299)

            q, k, v [S, E] -> Reshape [S, H, D] -> Permute [H, S, D]
            MatMul(q, k^T) -> Scale -> (+ causal mask) -> ChannelwiseSoftmax -> MatMul(., v)
            -> Permute [S, H, D] -> Reshape [S, E]

        becomes one call of ``ops.attention`` placed in the last Reshape: the layers between
        are not executed and the [H, S, S] scores are never formed.  When q, k and v are the
        three slices of one projection the packed entry point is used (one gradient tensor
        for the projection).  Dropout on the probabilities, extra biases, non-causal masks
        and protected (objective / metric) layers keep the layer-by-layer path."""
        if self.distconv is not None and getattr(self.distconv, "channel_groups", 1) > 1:
            return          # the attention chain is partitioned over tokens: keep its layers apart
        if os.environ.get("LBANN_DISABLE_ATTENTION_FUSION"):
            return
        protected = {n for n, _ in self.objective_terms} | {m.layer_name for m in self.metrics
                                                            if getattr(m, "layer_name", None)}

        def only_child(l, kind=None):
            if len(l.children) != 1 or l.name in protected:
                return None
            c = l.children[0]
            return c if (kind is None or c.type == kind) else None

        def heads_source(l):
            """l = Permute([1,0,2]) of Reshape([S, H, D]) of x  ->  (x, H, D, [layers])"""
            if l.type != "permute" or list(l.axes) != [1, 0, 2] or len(l.children) != 1 or l.name in protected:
                return None
            r = l.parents[0]
            if r.type != "reshape" or len(r.out_dims[0]) != 3 or len(r.children) != 1 or r.name in protected:
                return None
            S, H, D = r.out_dims[0]
            if tuple(r.in_dims[0]) != (S, H * D):
                return None
            return r.parents[0], H, D, [r, l]

        for sm in self.layers:
            if sm.type != "channelwise_softmax" or not sm.parents or sm.name in protected:
                continue
            scale = getattr(sm, "fused_scale", None)
            causal = getattr(sm, "fused_causal", None)
            cur = sm.parents[0]
            between = []
            ok = True
            while cur.type == "operator_layer":
                if not getattr(cur, "fused_into_child", False) or len(cur.children) != 1:
                    ok = False
                    break
                between.append(cur)
                cur = cur.parents[0]
            scores = cur
            if not ok or scores.type != "matmul" or scores.ta or not scores.tb or only_child(scores) is None:
                continue
            ctxl = only_child(sm, "matmul")
            if ctxl is None or ctxl.ta or ctxl.tb or ctxl.parents[0] is not sm:
                continue
            merge = only_child(ctxl, "permute")
            if merge is None or list(merge.axes) != [1, 0, 2]:
                continue
            out = only_child(merge, "reshape")
            if out is None or len(out.out_dims[0]) != 2:
                continue
            qs, ks, vs = heads_source(scores.parents[0]), heads_source(scores.parents[1]), \
                heads_source(ctxl.parents[1])
            if qs is None or ks is None or vs is None:
                continue
            H, D = qs[1], qs[2]
            if (ks[1], ks[2]) != (H, D) or (vs[1], vs[2]) != (H, D) or tuple(out.out_dims[0])[1] != H * D:
                continue
            Sq, Sk = scores.out_dims[0][-2], scores.out_dims[0][-1]
            if causal is not None and (causal != Sk or Sq != Sk):
                continue
            # only shapes that the tcgen05 kernels cover are rerouted (csrc/attention_tc.cu)
            if not os.environ.get("LBANN_FORCE_ATTENTION_FUSION") and (
                    self.device.type != "cuda" or D != 128 or Sq % 128 or Sk % 128
                    or self.default_dtype not in (torch.float16, torch.bfloat16)):
                continue
            mask_layers = [b for b in between if len(b.parents) == 2]
            if causal is None and mask_layers:
                continue            # an additive mask that is not the causal one
            dead = between + [scores, sm, ctxl, merge] + qs[3] + ks[3] + vs[3]
            for b in mask_layers:
                # the constant mask tensor itself is not needed either when nobody else reads it
                w = b.parents[1]
                if len(w.children) == 1:
                    dead.append(w)
            srcs = [qs[0], ks[0], vs[0]]
            packed = slice_layer = None
            if all(x.type == "identity" and len(x.children) == 1 and x.name not in protected for x in srcs):
                sl = srcs[0].parents[0]
                if (sl.type == "slice" and all(x.parents[0] is sl for x in srcs)
                        and [c.name for c in sl.children] == [x.name for x in srcs]
                        and sl.points == [0, H * D, 2 * H * D, 3 * H * D] and sl.name not in protected
                        and sl.axis == len(sl.in_dims[0]) - 1):
                    packed, slice_layer = sl.parents[0], sl
                    dead += srcs + [sl]
            for l in dead:
                l.dead = True
            out.attention = {"packed": packed.name if packed is not None else None,
                             "q": srcs[0].name, "k": srcs[1].name, "v": srcs[2].name,
                             "heads": H, "scale": float(scale) if scale is not None else 1.0,
                             "causal": causal is not None}
            out.attention_sources = (packed, slice_layer) if packed is not None else tuple(srcs)

    def _attention_forward(self, layer, acts):
        from ..ops import attention as att
        a = layer.attention
        if a["packed"] is not None:
            src, consumer = layer.attention_sources
            qkv = acts[src.name][self._slot(src, consumer)]
            y = att.attention_packed(layer.cast_in(qkv), a["heads"], a["scale"], a["causal"])
        else:
            q, k, v = (layer.cast_in(acts[s.name][self._slot(s, s.children[0])])
                       for s in layer.attention_sources)
            y = att.attention(q, k, v, a["heads"], a["scale"], a["causal"])
        return [y.reshape(y.shape[0], *layer.out_dims[0])]

    # ------------------------------------------------------------------ execution
    def forward_prop(self, inputs: Dict[str, torch.Tensor], mode: str = "training",
                     global_mini_batch_size: Optional[int] = None, mini_batch_offset: int = 0):
        training = mode == "training"
        self.current_inputs = inputs
        first = next(iter(inputs.values())) if inputs else None
        self.current_mini_batch_size = int(first.shape[0]) if first is not None else 0
        dp = self.parallel.dp_size if self.parallel is not None else 1
        self._global_mb = global_mini_batch_size or self.current_mini_batch_size * dp
        self._global_mb_given = bool(global_mini_batch_size)
        self._mb_offset = mini_batch_offset
        acts = {}
        self.acts = acts          # visible to callbacks while it fills up
        self._mean_cache = {}
        cbs = self.callbacks
        occurrence = defaultdict(int)
        sg = self.subgrid
        if sg is not None:
            sg.dangling.clear()
            base_mb = self.current_mini_batch_size
        for layer in self.layers:
            if getattr(layer, "dead", False):        # folded into a fused consumer
                acts[layer.name] = [None] * max(len(layer.out_dims), 1)
                continue
            if getattr(layer, "attention", None) is not None:
                acts[layer.name] = self._attention_forward(layer, acts)
                continue
            xs = []
            occ_local = defaultdict(int)
            for pn in layer.parent_names:
                parent = self.layers_by_name[pn]
                k = occ_local[pn]
                occ_local[pn] += 1
                xs.append(acts[pn][self._slot(parent, layer, k)])
            if self.distconv is not None:
                xs = self.distconv.adapt_inputs(self, layer, xs)
            if sg is not None:
                # sub-graph parallelism: bring every input to this layer's grid (collective
                # over the trainer), then only the grid's ranks compute
                tag = layer.grid_tag
                moved = []
                for k, (pn, x) in enumerate(zip(layer.parent_names, xs)):
                    parent = self.layers_by_name[pn]
                    if parent.grid_tag != tag:
                        slot = self._slot(parent, layer, 0)
                        dims = parent.out_dims[slot] if slot < len(parent.out_dims) else parent.out_dims[0]
                        dt = x.dtype if x is not None else self._act_dtype(parent)
                        x = sg.transfer(x, parent.grid_tag, tag, self._global_mb, dims, dt,
                                        f"{pn}>{layer.name}#{k}")
                    moved.append(x)
                xs = moved
                if not sg.member(tag):
                    acts[layer.name] = [None] * max(len(layer.out_dims), 1)
                    continue
                self.current_mini_batch_size = sg.local_count(tag, self._global_mb) if layer.type != "input" \
                    else base_mb
            for cb in cbs:
                cb.on_layer_forward_begin(self, layer, mode)
            if self.layer_timing:
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
            pt = self._phase_timer
            if pt is not None:
                th = time.perf_counter()
            ys = layer.forward(xs, training)
            if pt is not None:          # host time of the layer's forward (no synchronisation)
                pt.layer_host[layer.name] += time.perf_counter() - th
            if self.layer_timing or self.sync_layers:
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                if self.layer_timing:
                    layer.fp_time += time.perf_counter() - t0
            acts[layer.name] = ys
            if self.distconv is not None:
                self.distconv.note_outputs(self, layer)
            for cb in cbs:
                cb.on_layer_forward_end(self, layer, mode)
        if sg is not None:
            self.current_mini_batch_size = base_mb
        self.acts = acts
        return acts

    def _layer_mean(self, layer_name: str) -> torch.Tensor:
        """Sum over the local mini-batch divided by the global mini-batch size."""
        hit = self._mean_cache.get(layer_name)      # objective term and metric often coincide
        if hit is not None:
            return hit
        layer = self.layers_by_name[layer_name]
        y = self.acts[layer_name][0] if self.acts[layer_name] else self.acts[layer.parent_names[0]][0]
        if y is None:        # computed on a sub-grid this rank does not belong to
            val = torch.zeros((), device=self.device)
            self._mean_cache[layer_name] = val
            return val
        val = y.float().sum() / float(self._global_mb)
        self._mean_cache[layer_name] = val
        return val

    def local_objective(self) -> torch.Tensor:
        total = None
        for name, scale in self.objective_terms:
            v = self._layer_mean(name) * scale
            total = v if total is None else total + v
        if total is None:
            total = torch.zeros((), device=self.device)
        if self.subgrid is not None:
            # tensors that this rank handed to another grid and does not consume itself: a zero
            # term keeps them in the autograd graph, so that this rank takes part in the
            # exchanges of the backward pass
            for d in self.subgrid.dangling:
                total = total + d.float().sum() * 0.0
        return total

    def _act_dtype(self, layer) -> torch.dtype:
        dt = layer.dtype or self.default_dtype
        return dt if isinstance(dt, torch.dtype) else self.default_dtype

    def l2_value(self) -> torch.Tensor:
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        for scale, names in self.l2_terms:
            for n in names:
                w = self.weights_by_name.get(n)
                if w is not None:
                    total = total + 0.5 * scale * (w.handle.master.detach().float() ** 2).sum()
        return total

    def record_statistics(self, mode: str, local_obj: torch.Tensor):
        st = self.stats[mode]
        n = self._global_mb
        with torch.no_grad():
            st.obj_sum.add_(local_obj.detach(), alpha=n)
            st.samples += n
            for i, m in enumerate(self.metrics):
                if getattr(m, "layer_name", None):
                    st.metric_sums[i].add_(self._layer_mean(m.layer_name).detach(), alpha=n)

    def clear_gradients(self):
        self.arena.zero_grad()

    def sync_optimizer_state(self):
        """Collective over the trainer: optimizer state that the ranks hold in shards (the
        sharded update of data-parallel GPU runs) becomes whole on every rank."""
        if self.parallel is not None and self.arena is not None:
            self.parallel.sync_optimizer_state(self)

    def snapshot_state(self) -> dict:
        """In-memory copy of everything a training step changes on this rank: weights (fp32
        values and their 16-bit copies), optimizer state and step counters, the loss-scale
        schedule.  ``restore_state`` writes it back into the same buffers, so a captured
        graph stays valid.  The in-memory counterpart of a checkpoint; the reference keeps
        such copies of a model's weights for tournaments (src/execution_algorithms/ltfb/
        regularized_evolution.cpp) and for its check_* callbacks."""
        a = self.arena
        snap = {}
        for k in ("master", "state0", "state1", "compute", "step_dev"):
            v = getattr(a, k, None)
            if v is not None:
                snap[k] = v.detach().clone()
        snap["slot_steps"] = [s.step_count for s in a.slots]
        snap["slot_extra"] = [{k: v.clone() for k, v in s.extra.items()} for s in a.slots]
        if self._amp_state is not None:
            snap["amp_state"] = self._amp_state.clone()
        snap["amp_host"] = (self._amp_scale_host, getattr(self, "_amp_good_steps", 0))
        return snap

    def restore_state(self, snap: dict) -> None:
        a = self.arena
        for k in ("master", "state0", "state1", "compute", "step_dev"):
            v = getattr(a, k, None)
            if k in snap and v is not None:
                v.copy_(snap[k])
            elif v is not None and k in ("state0", "state1"):
                v.zero_()          # allocated after the snapshot was taken
            elif v is not None and k == "step_dev":
                v.zero_()
        for s, n, e in zip(a.slots, snap["slot_steps"], snap["slot_extra"]):
            s.step_count = n
            for k in list(s.extra):
                if k in e:
                    s.extra[k].copy_(e[k])
                else:
                    del s.extra[k]
        if "amp_state" in snap and self._amp_state is not None:
            self._amp_state.copy_(snap["amp_state"])
        self._amp_scale_host, self._amp_good_steps = snap["amp_host"]

    def backward_prop(self, local_obj: torch.Tensor):
        for cb in self.callbacks:
            cb.on_backward_prop_begin(self)
        if local_obj.requires_grad:
            if not self.amp_enabled:
                local_obj.backward()
            elif self.device.type == "cuda":
                (local_obj * self._amp_device_state()[0]).backward()     # no host read of the scale
            else:
                (local_obj * self._amp_scale_host).backward()
        if self.parallel is not None:
            self.parallel.sync_gradients(self)
        for cb in self.callbacks:
            cb.on_backward_prop_end(self)

    @property
    def amp_scale(self) -> float:
        """Current loss scale (reads the device copy when the schedule runs there)."""
        if self._amp_state is not None:
            return float(self._amp_state[0].item())
        return self._amp_scale_host

    @amp_scale.setter
    def amp_scale(self, value: float):
        self._amp_scale_host = float(value)
        if self._amp_state is not None:
            self._amp_state[0] = float(value)
            self._amp_state[1] = 1.0 / float(value)

    def _amp_device_state(self) -> torch.Tensor:
        if self._amp_state is None:
            s = self._amp_scale_host
            self._amp_state = torch.tensor([s, 1.0 / s, 0.0, 0.0, 1.0 / s], dtype=torch.float32,
                                           device=self.device)
        return self._amp_state

    def update_weights(self) -> bool:
        """Returns False when the step was skipped (AMP overflow)."""
        for cb in self.callbacks:
            cb.on_optimize_begin(self)
        inv = 1.0
        skip_flag = None
        skipped = False
        amp_inv = None
        if self.amp_enabled:
            # the reference's schedule: src/models/model.cpp:1796-1824
            flag = torch.zeros(1, dtype=torch.int32, device=self.device)
            if self.device.type == "cuda":
                # Overflow flag, loss scale and its schedule all stay on the device: the fused
                # optimizer reads the flag and skips the update by itself, so a step needs no
                # host synchronisation (and can be captured as a graph).
                st = self._amp_device_state()
                # the check only reads; the optimizer unscales in registers (st[4] = inverse of
                # the scale that this step's gradients carry)
                self.arena.unscale_and_check(1.0, flag, write_back=False, inv_scale_dev=st[1:2])
                amp_inv = st[4:5]
                reduced = None
                if self.parallel is not None and self.parallel.world_size > 1:
                    reduced = flag.float()
                    self.parallel.allreduce_max_inplace(reduced)
                from ..ops import optim as _optim
                _optim.amp_update(st, reduced, flag, self.amp_growth, self.amp_backoff, self.amp_interval)
                skip_flag = flag
            else:
                self.arena.unscale_and_check(1.0 / self._amp_scale_host, flag, write_back=True)
                if self.parallel is not None:
                    self.parallel.allreduce_max_inplace(flag)
                overflow = bool(int(flag.item()))
                skipped = overflow
                if overflow:
                    self._amp_scale_host *= self.amp_backoff
                    self._amp_good_steps = 0
                    self._amp_skipped += 1
                    if self._amp_skipped >= 10 and (self.comm is None or self.comm.am_world_master()):
                        print(f"WARNING: {self._amp_skipped} consecutive steps skipped by automatic "
                              f"mixed precision; loss scale is now {self._amp_scale_host}")
                else:
                    self._amp_skipped = 0
                    self._amp_good_steps += 1
                    if self._amp_good_steps >= self.amp_interval:
                        self._amp_scale_host *= self.amp_growth
                        self._amp_good_steps = 0
            if skipped:
                return False
        self.arena.step(inv, skip_flag if self.device.type == "cuda" else None, inv_scale_dev=amp_inv)
        for w in self.weights:
            w.handle.bump()
        for cb in self.callbacks:
            cb.on_optimize_end(self)
        return True

    def train_step(self, inputs, global_mini_batch_size=None, mini_batch_offset=0):
        """clear grads -> forward -> objective -> backward (+ gradient sync) -> update.
        With the ``use_cuda_graph`` option the step is captured once per input signature as
        a CUDA graph and replayed afterwards."""
        if self._graph_mode is None:
            self._graph_mode = self._graph_capable()
        if self._graph_mode:
            return self._train_step_graph(inputs, global_mini_batch_size, mini_batch_offset)
        return self._train_step_eager(inputs, global_mini_batch_size, mini_batch_offset)

    # ------------------------------------------------------------------ CUDA-graph replay
    _IN_STEP_HOOKS = ("on_forward_prop_begin", "on_forward_prop_end", "on_layer_forward_begin",
                      "on_layer_forward_end", "on_backward_prop_begin", "on_backward_prop_end",
                      "on_optimize_begin", "on_optimize_end")

    def _graph_capable(self) -> bool:
        """Graph replay is used when asked for, on a GPU, and when nothing needs the host
        inside a step: no callback overrides an in-step hook, no per-layer timing."""
        from ..callbacks.base import ExecCallback
        from ..utils import options as _opts
        if self.device.type != "cuda" or not (_opts.current().get_bool("use_cuda_graph")
                                              or os.environ.get("LBANN_CUDA_GRAPH") == "1"):
            return False
        if self.layer_timing or self.sync_layers or (self._phase_timer is not None and not self._phase_graphs):
            return False
        for cb in self.callbacks:
            for h in self._IN_STEP_HOOKS:
                if getattr(type(cb), h, None) is not getattr(ExecCallback, h):
                    return False
        # layers whose output depends on a host-side value that changes from step to step
        # (position in the epoch, host random streams, user code)
        if any(l.type in self._HOST_STATE_LAYERS for l in self.layers):
            return False
        # hypergradient Adam moves its learning rate on the host every step
        if any(s.kind == "hypergradient_adam" for s in self.arena.slots):
            return False
        return True

    _HOST_STATE_LAYERS = frozenset({"mini_batch_index", "dropout", "selu_dropout", "bernoulli", "gaussian",
                                    "uniform", "dist_embedding", "external", "python"})

    @staticmethod
    def _copy_into_static(static: torch.Tensor, v: torch.Tensor):
        """Copy a step's input into the graph's input buffer with a copy KERNEL (a device
        memcpy would queue behind the next mini-batch's upload on the copy engines: measured
        +1.4 ms per step end to end)."""
        if v.data_ptr() == static.data_ptr():
            return
        if (v.dtype == static.dtype and v.is_contiguous() and static.is_contiguous()
                and v.is_cuda and v.element_size() in (2, 4) and v.shape == static.shape):
            # ``copy_`` between dense tensors of one dtype is a device memcpy; an element-wise
            # kernel on the bit pattern is the same copy on the SMs (25 us for 69 MB)
            bits = torch.int16 if v.element_size() == 2 else torch.int32
            torch.bitwise_or(v.view(bits), 0, out=static.view(bits))
        else:
            static.copy_(v)

    def _train_step_graph(self, inputs, gmb, offset):
        key = (tuple((k, tuple(v.shape), v.dtype) for k, v in sorted(inputs.items())), gmb)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._graphs[key] = {"warm": 0}
        if "graph" not in entry:
            if entry["warm"] < 3:
                # lazy allocations, symmetric buffers, tensor maps and optimizer tables are
                # created by ordinary steps first
                entry["warm"] += 1
                return self._train_step_eager(inputs, gmb, offset)
            static = {k: torch.empty_like(v) for k, v in inputs.items()}
            for k, v in inputs.items():
                self._copy_into_static(static[k], v)
            samples0 = self.stats["training"].samples
            counts0 = [s.step_count for s in self.arena.slots]
            launches0 = native.launches()
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            try:
                if self._phase_graphs:
                    graph = self._capture_phase_graphs(static, gmb, offset)
                    out = self.last_objective
                else:
                    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                        out = self._train_step_eager(static, gmb, offset)
            except Exception as e:      # something in this model cannot be captured
                self._graph_mode = False
                self._graphs.clear()
                self.stats["training"].samples = samples0
                for s, c in zip(self.arena.slots, counts0):
                    s.step_count = c
                native.count_launch(launches0 - native.launches())
                if self.comm is None or self.comm.am_world_master():
                    print(f"WARNING: the training step could not be captured as a CUDA graph ({e}); "
                          "kernels are launched from the host", flush=True)
                torch.cuda.synchronize(self.device)
                return self._train_step_eager(inputs, gmb, offset)
            # capture executes nothing: undo the host-side bookkeeping it did, replay does it
            self.stats["training"].samples = samples0
            for s, c in zip(self.arena.slots, counts0):
                s.step_count = c
            entry.update(graph=graph, static=static, out=out, acts=self.acts,
                         launches=native.launches() - launches0, samples=self._global_mb)
            native.count_launch(-entry["launches"])
        else:
            for k, v in inputs.items():
                self._copy_into_static(entry["static"][k], v)
        # hyper-parameters changed by callbacks (learning-rate schedules) reach the captured
        # optimizer kernel through its device-side table, refreshed here when they change
        self.arena._segments()
        entry["graph"].replay()
        self.stats["training"].samples += entry["samples"]
        for s in self.arena.slots:
            if s.kind != "none":
                s.step_count += 1
        native.count_launch(entry["launches"])
        self.acts = entry["acts"]
        self.current_inputs = entry["static"]
        self.last_objective = entry["out"]
        return self.last_objective

    def _capture_phase_graphs(self, static, gmb, offset):
        """The step as three graphs in one memory pool; ``replay()`` of the returned object
        runs them in order with timing events between (see LBANN_PHASE_TIMING=graph)."""
        model = self
        pool = torch.cuda.graph_pool_handle()
        graphs = [torch.cuda.CUDAGraph() for _ in range(3)]
        pt, self._phase_timer = self._phase_timer, None       # no event records inside a capture
        try:
            with torch.cuda.graph(graphs[0], pool=pool, capture_error_mode="thread_local"):
                self.clear_gradients()
                self.forward_prop(static, "training", gmb, offset)
                obj = self.local_objective()
                self.last_objective = obj.detach()
                self.record_statistics("training", obj)
            with torch.cuda.graph(graphs[1], pool=pool, capture_error_mode="thread_local"):
                self.backward_prop(obj)
            with torch.cuda.graph(graphs[2], pool=pool, capture_error_mode="thread_local"):
                self.update_weights()
        finally:
            self._phase_timer = pt

        class _Three:
            def replay(self_inner):
                pt.mark("start")
                for g, name in zip(graphs, ("forward", "backward+sync", "update")):
                    g.replay()
                    pt.mark(name)
        return _Three()

    def _train_step_eager(self, inputs, global_mini_batch_size=None, mini_batch_offset=0):
        pt = self._phase_timer
        if pt is not None:
            pt.mark("start")
        self.clear_gradients()
        for cb in self.callbacks:
            cb.on_forward_prop_begin(self, "training")
        self.forward_prop(inputs, "training", global_mini_batch_size, mini_batch_offset)
        for cb in self.callbacks:
            cb.on_forward_prop_end(self, "training")
        obj = self.local_objective()
        self.last_objective = obj.detach()
        self.record_statistics("training", obj)
        if pt is not None:
            pt.mark("forward")
        self.backward_prop(obj)
        if pt is not None:
            pt.mark("backward+sync")
        self.update_weights()
        if pt is not None:
            pt.mark("update")
        return self.last_objective

    class _PhaseTimer:
        """Per-phase device and host times of the training step (LBANN_PHASE_TIMING=1):
        CUDA events between the phases plus host timestamps, summarised by ``report``."""

        def __init__(self, device):
            self.device, self.events, self.host, self.steps = device, [], [], 0
            self.layer_host = defaultdict(float)
            self.dev_ms, self.host_ms = defaultdict(float), defaultdict(float)

        def mark(self, name):
            ev = None
            if self.device.type == "cuda":
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
            self.events.append((name, ev, time.perf_counter()))
            if name == "update":
                self.steps += 1
                if self.steps % 16 == 0:
                    self.flush()

        def flush(self):
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            prev = None
            for name, ev, t in self.events:
                if name != "start" and prev is not None:
                    if ev is not None:
                        self.dev_ms[name] += prev[1].elapsed_time(ev)
                    self.host_ms[name] += (t - prev[2]) * 1e3
                prev = (name, ev, t)
            self.events = []

        def report(self):
            self.flush()
            n = max(self.steps, 1)
            out = {k: (round(self.dev_ms[k] / n, 3), round(self.host_ms[k] / n, 3)) for k in self.host_ms}
            top = sorted(self.layer_host.items(), key=lambda kv: -kv[1])[:12]
            out["forward host ms by layer"] = {k: round(v * 1e3 / n, 3) for k, v in top}
            return out

    @torch.no_grad()
    def evaluate_step(self, inputs, mode="validation", global_mini_batch_size=None,
                      mini_batch_offset=0):
        for cb in self.callbacks:
            cb.on_forward_prop_begin(self, mode)
        if self.distconv is not None:
            # forward-only steps have no gradient reduction between them: the ranks meet here,
            # so that no rank sends halo planes into a tensor a neighbour still reads
            self.distconv.step_barrier()
        self.forward_prop(inputs, mode, global_mini_batch_size, mini_batch_offset)
        for cb in self.callbacks:
            cb.on_forward_prop_end(self, mode)
        obj = self.local_objective()
        self.last_objective = obj.detach()
        self.record_statistics(mode, obj)
        return self.last_objective

    # ------------------------------------------------------------------ reporting
    def reduce_statistics(self, mode: str):
        """-> (mean objective incl. L2, [metric means], samples) over the trainer."""
        st = self.stats[mode]
        vals = torch.stack([st.obj_sum] + st.metric_sums) if st.metric_sums else st.obj_sum.reshape(1)
        vals = vals.clone()
        if self.parallel is not None and self.parallel.dp_size > 1:
            self.parallel.allreduce_sum_inplace(vals)
        n = max(st.samples, 1)
        vals = (vals / n).tolist()
        obj = vals[0] + float(self.l2_value())
        mets = vals[1:]
        for i, m in enumerate(self.metrics):
            if not getattr(m, "layer_name", None):
                mets[i] = m.evaluate(self, mode)
            elif m.unit == "%":
                mets[i] *= 100.0     # layer metrics in percent (src/metrics/layer_metric.cpp)
        return obj, mets, st.samples

    def reset_statistics(self, mode: str):
        self.stats[mode].reset()

    def describe(self) -> str:
        lines = [f"model {self.name}: {len(self.layers)} layers, {len(self.weights)} weights, "
                 f"{sum(w.slot.count for w in self.weights)} parameters"]
        lines += ["  " + l.describe() for l in self.layers]
        return "\n".join(lines)
