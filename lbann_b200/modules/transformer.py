"""Attention and sequence-encoding modules (``lbann.modules.transformer``).

Tensors are ``[sequence, embed]`` per sample, as in the reference
(python/lbann/modules/transformer/attention.py:9-424, encoding.py:9-357).  The attention
module emits the projection -> head split -> QK^T -> scale (+ bias / mask) -> softmax ->
dropout -> PV -> merge -> projection layer chain; the executor recognises the
``<name>_instance<k>_`` scores..context span and runs it as one fused attention op when
the inputs are on a GPU (ops/attention.py).
"""
from __future__ import annotations

import math

import numpy as np

from ..frontend import core as L
from .base import Module


class MultiheadAttention(Module):
    """Scaled dot-product attention over ``num_heads`` heads of size embed_dim / num_heads."""

    global_count = 0

    def __init__(self, embed_dim, num_heads, self_attention=False, batch_heads=True, dropout=0.0,
                 subgraph_branches=0, bias=None, positional_encoding=None, name=None):
        super().__init__()
        MultiheadAttention.global_count += 1
        if embed_dim % num_heads:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.instance = 0
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.head_dim = embed_dim // num_heads
        self.dropout, self.bias = dropout, bias
        self.positional_encoding = positional_encoding
        self.self_attention = self_attention
        self.subgraph_branches = subgraph_branches
        if subgraph_branches > 0 and num_heads % subgraph_branches:
            raise ValueError("number of heads must be divisible by the number of branches")
        self.separate_heads = subgraph_branches > 0 or not batch_heads
        self.name = name or f"multiheadattention{MultiheadAttention.global_count}"

        def pair(tag):
            return [L.Weights(initializer=L.GlorotNormalInitializer(), name=f"{self.name}_{tag}_matrix"),
                    L.Weights(initializer=L.ConstantInitializer(value=0), name=f"{self.name}_{tag}_bias")]

        if self_attention:
            self.qkv_weights = pair("qkv")
        else:
            self.query_weights, self.key_weights, self.value_weights = pair("query"), pair("key"), pair("value")
        self.output_weights = pair("output")

    # ------------------------------------------------------------------ projections
    def _project(self, queries, keys, values, name, seqlen=None):
        E = self.embed_dim
        if self.self_attention:
            qkv = L.ChannelwiseFullyConnected(queries, weights=self.qkv_weights, output_channel_dims=[3 * E],
                                              name=f"{name}_qkv_fc", bias=True, transpose=False)
            sl = L.Slice(qkv, axis=1, slice_points=[0, E, 2 * E, 3 * E], name=f"{name}_qkv_slice")
            q, k, v = (L.Identity(sl, name=f"{name}_{t}_fc") for t in ("queries", "keys", "values"))
        else:
            q = L.ChannelwiseFullyConnected(queries, weights=self.query_weights, output_channel_dims=[E],
                                            name=f"{name}_queries_fc")
            k = L.ChannelwiseFullyConnected(keys, weights=self.key_weights, output_channel_dims=[E],
                                            name=f"{name}_keys_fc")
            v = L.ChannelwiseFullyConnected(values, weights=self.value_weights, output_channel_dims=[E],
                                            name=f"{name}_values_fc")
        if self.positional_encoding is not None:
            q, k, v = self.positional_encoding.apply_layer(q, k, v, seqlen)
        return q, k, v

    def forward(self, queries, keys, values, mask=None, seqlen=None):
        """``mask``: additive ``[heads or 1, seq_q, seq_k]`` tensor applied before the
        softmax (e.g. -1e9 above the diagonal for causal attention)."""
        self.instance += 1
        name = f"{self.name}_instance{self.instance}"
        q, k, v = self._project(queries, keys, values, name, seqlen)
        H, D = self.num_heads, self.head_dim
        if self.separate_heads:
            ctx = self._separate(q, k, v, mask, name)
        else:
            # [seq, E] -> [seq, H, D] -> [H, seq, D]
            def heads(x, tag):
                x = L.Reshape(x, dims=[-1, H, D], name=f"{name}_{tag}_reshape")
                return L.TensorPermute(x, axes=[1, 0, 2], name=f"{name}_{tag}_heads")

            qh, kh, vh = heads(q, "queries"), heads(k, "keys"), heads(v, "values")
            scores = L.MatMul(qh, kh, transpose_b=True, name=f"{name}_scores")
            scores = L.Scale(scores, constant=1.0 / math.sqrt(D), name=f"{name}_scale")
            if self.bias is not None:
                scores = L.Add(scores, self.bias, name=f"{name}_bias")
            if mask is not None:
                scores = L.Add(scores, mask, name=f"{name}_mask")
            probs = L.ChannelwiseSoftmax(scores, dim=-1, single_dim_mode=True, name=f"{name}_softmax")
            if self.dropout > 0:
                probs = L.Dropout(probs, keep_prob=1 - self.dropout, name=f"{name}_drop")
            ctx = L.MatMul(probs, vh, name=f"{name}_context")
            ctx = L.TensorPermute(ctx, axes=[1, 0, 2], name=f"{name}_merge")
            ctx = L.Reshape(ctx, dims=[-1, self.embed_dim], name=f"{name}_merge_reshape")
        return L.ChannelwiseFullyConnected(ctx, weights=self.output_weights,
                                           output_channel_dims=[self.embed_dim], name=name)

    def _separate(self, q, k, v, mask, name):
        """One small attention per head (the reference's non-batched mode).  With
        ``subgraph_branches`` = B > 0 the heads are dealt in blocks onto the sub-grids 1..B
        (grid tags; python/lbann/modules/attention_allsubgraph.py does the same with its
        branch tags): each sub-grid computes its heads for the whole mini-batch, the slices
        and the concatenation run on the whole trainer and move the tensors between grids."""
        H, D = self.num_heads, self.head_dim
        B = self.subgraph_branches
        pts = [i * D for i in range(H + 1)]
        qs = L.Slice(q, axis=1, slice_points=pts, name=f"{name}_queries_slice")
        ks = L.Slice(k, axis=1, slice_points=pts, name=f"{name}_keys_slice")
        vs = L.Slice(v, axis=1, slice_points=pts, name=f"{name}_values_slice")
        outs = []
        for h in range(H):
            hn = f"{name}_head{h}"
            kw = {"grid_tag": 1 + h // (H // B)} if B > 0 else {}
            qh, kh, vh = (L.Identity(s, name=f"{hn}_{t}", **kw) for s, t in ((qs, "q"), (ks, "k"), (vs, "v")))
            y = L.MatMul(qh, kh, transpose_b=True, name=f"{hn}_matmul", **kw)
            y = L.Scale(y, constant=1.0 / math.sqrt(D), name=f"{hn}_scale", **kw)
            if mask is not None:       # a [seq_q, seq_k] mask shared by the heads in this mode
                y = L.Add(y, mask, name=f"{hn}_mask", **kw)
            y = L.ChannelwiseSoftmax(y, name=f"{hn}_softmax", **kw)
            if self.dropout > 0:
                y = L.Dropout(y, keep_prob=1 - self.dropout, name=f"{hn}_drop", **kw)
            outs.append(L.MatMul(y, vh, name=f"{hn}_context", **kw))
        return L.Concatenation(outs, axis=1, name=f"{name}_heads_concat", **({"grid_tag": 0} if B > 0 else {}))


class SequenceEncoding:
    """Interface of positional encodings: ``apply_input`` on the embedded sequence and
    ``apply_layer`` on the per-layer query / key / value projections."""

    def apply_input(self, x, length):
        return x

    def apply_layer(self, q, k, v, length=None):
        return q, k, v


def _constant_table(array: np.ndarray, name: str):
    w = L.Weights(initializer=L.ValueInitializer(values=array.astype(np.float32).reshape(-1).tolist()),
                  optimizer=L.NoOptimizer(), name=name)
    return L.WeightsLayer(weights=w, dims=list(array.shape), name=name + "_layer")


class PositionalEncoding(SequenceEncoding):
    """Sinusoidal encoding added to the input embeddings (Vaswani et al., section 3.5)."""

    global_count = 0

    def __init__(self, embed_dim, dropout=0.0, name=None):
        PositionalEncoding.global_count += 1
        self.embed_dim, self.dropout = embed_dim, dropout
        self.name = name or f"positionalencoding{PositionalEncoding.global_count}"
        self._cache = {}
        self.instance = 0

    def _table(self, length):
        if length not in self._cache:
            pos = np.arange(length)[:, None]
            i = np.arange(self.embed_dim)[None, :]
            angle = pos / np.power(10000.0, (2 * (i // 2)) / self.embed_dim)
            tab = np.where(i % 2 == 0, np.sin(angle), np.cos(angle))
            self._cache[length] = _constant_table(tab, f"{self.name}_table{length}")
        return self._cache[length]

    def apply_input(self, x, length):
        self.instance += 1
        y = L.Add(x, self._table(length), name=f"{self.name}_instance{self.instance}_add")
        if self.dropout > 0:
            y = L.Dropout(y, keep_prob=1 - self.dropout, name=f"{self.name}_instance{self.instance}_drop")
        return y


class LearnedInputEncoding(SequenceEncoding):
    """Trainable position embeddings added to the token embeddings (GPT style)."""

    global_count = 0

    def __init__(self, embed_dim, max_sequence_length, dropout=0.0, name=None):
        LearnedInputEncoding.global_count += 1
        self.embed_dim, self.max_len, self.dropout = embed_dim, max_sequence_length, dropout
        self.name = name or f"learnedinputencoding{LearnedInputEncoding.global_count}"
        self.weights = L.Weights(initializer=L.NormalInitializer(standard_deviation=0.01),
                                 name=f"{self.name}_positions")
        self.instance = 0

    def apply_input(self, x, length):
        self.instance += 1
        name = f"{self.name}_instance{self.instance}"
        table = L.WeightsLayer(weights=self.weights, dims=[self.max_len, self.embed_dim],
                               name=f"{name}_table")
        if length != self.max_len:
            table = L.Identity(L.Slice(table, axis=0, slice_points=[0, length], name=f"{name}_slice"))
        y = L.Add(x, table, name=f"{name}_add")
        if self.dropout > 0:
            y = L.Dropout(y, keep_prob=1 - self.dropout, name=f"{name}_drop")
        return y


class RotaryPositionalEmbedding(SequenceEncoding):
    """Rotary position embedding (Su et al., arXiv:2104.09864) applied to the per-layer
    queries and keys (and, with ``embed_values``, the values): each head's vector is rotated
    pairwise by position-dependent angles, ``x cos + rotate_half(x) sin``.  The cos / sin
    tables are constant weights of shape ``[sequence, heads * freq_dim]``
    (python/lbann/modules/transformer/encoding.py:226-357)."""

    global_count = 0

    def __init__(self, freq_dim, max_sequence_length, num_heads, embed_values=False, theta=10000.0,
                 name=None):
        RotaryPositionalEmbedding.global_count += 1
        if freq_dim % 2:
            raise ValueError(f"rotary embedding needs an even number of frequencies, got {freq_dim}")
        self.name = name or f"rope{RotaryPositionalEmbedding.global_count}"
        self.dim, self.max_len, self.num_heads = freq_dim, max_sequence_length, num_heads
        self.embed_values, self.theta = embed_values, theta
        self.instance = 0
        inv_freq = 1.0 / theta ** (np.arange(0, freq_dim, 2) / freq_dim)
        ang = np.outer(np.arange(max_sequence_length), inv_freq)
        ang = np.concatenate([ang, ang], axis=-1)
        self.cos = _constant_table(np.tile(np.cos(ang), num_heads), f"{self.name}_cos")
        self.sin = _constant_table(np.tile(np.sin(ang), num_heads), f"{self.name}_sin")

    def _rotate_half(self, x, length, name):
        H, P = self.num_heads, self.dim
        r = L.Reshape(x, dims=[length, H, P], name=f"{name}_split")
        s = L.Slice(r, axis=2, slice_points=[0, P // 2, P], name=f"{name}_halves")
        x1 = L.Identity(s, name=f"{name}_lo")
        x2 = L.Identity(s, name=f"{name}_hi")
        cat = L.Concatenation([L.Scale(x2, constant=-1.0, name=f"{name}_neg"), x1], axis=2,
                              name=f"{name}_cat")
        return L.Reshape(cat, dims=[length, H * P], name=f"{name}_merge")

    def _embed(self, x, length, cos, sin, name):
        rot = self._rotate_half(x, length, name)
        return L.Add(L.Multiply(x, cos, name=f"{name}_cos"), L.Multiply(rot, sin, name=f"{name}_sin"),
                     name=f"{name}_out")

    def apply_layer(self, q, k, v, length=None):
        length = length or self.max_len
        self.instance += 1
        base = f"{self.name}_instance{self.instance}"
        cos, sin = self.cos, self.sin
        if length != self.max_len:
            cos = L.Identity(L.Slice(cos, axis=0, slice_points=[0, length], name=f"{base}_cos_slice"))
            sin = L.Identity(L.Slice(sin, axis=0, slice_points=[0, length], name=f"{base}_sin_slice"))
        eq = self._embed(q, length, cos, sin, f"{base}_q")
        ek = self._embed(k, length, cos, sin, f"{base}_k")
        ev = self._embed(v, length, cos, sin, f"{base}_v") if self.embed_values else v
        return eq, ek, ev
