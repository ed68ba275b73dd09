"""RoBERTa encoder (Liu et al. 2019) from the front-end layers.

Follows the HuggingFace configuration vocabulary (``vocab_size``, ``hidden_size``,
``num_hidden_layers``, ``num_attention_heads``, ``intermediate_size``,
``max_position_embeddings``, ``type_vocab_size``, ``pad_token_id``, ``layer_norm_eps``,
``hidden_dropout_prob``, ``attention_probs_dropout_prob``) like the reference's model
(python/lbann/models/roberta.py); a sample is a sequence of ``seq_len`` token ids.

    cfg = RobertaConfig(vocab_size=50265, hidden_size=768, ...)
    model = RoBERTa(cfg, seq_len=128, load_weights="/path/to/npy")   # or load_weights=False
    hidden, pooled = model(token_ids)

Position ids skip padding tokens (``cumsum(ids != pad) * (ids != pad) + pad``).  Attention of
all heads of a layer runs as batched products; an optional ``attention_mask`` ([seq] of
0 / 1) is turned into an additive ``-10000`` mask on the key axis.  With ``load_weights`` set
to a directory every parameter ``<name>.npy`` is read from there (names as in the reference's
converted checkpoints, e.g. ``embeddings.word_embeddings.weight``,
``encoder.layer.0.attention.self.query.weight``).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional, Union

from ..frontend import core as L
from ..modules import Cumsum, Module


@dataclass
class RobertaConfig:
    vocab_size: int = 50265
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    hidden_act: str = "gelu"
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    max_position_embeddings: int = 514
    type_vocab_size: int = 1
    layer_norm_eps: float = 1e-5
    pad_token_id: int = 1
    position_embedding_type: str = "absolute"


class _Params:
    """Weights of the model by parameter name: fresh initialisers, or ``<dir>/<name>.npy``."""

    def __init__(self, load_weights: Union[bool, str, None]):
        self.dir = load_weights if isinstance(load_weights, str) else None
        if load_weights is True:
            self.dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pretrained_weights")

    def get(self, name: str, init=None):
        if self.dir is not None:
            f = os.path.join(self.dir, name + ".npy")
            if not os.path.isfile(f):
                raise ValueError(f"pretrained weight file does not exist: {f}")
            return L.Weights(initializer=L.NumpyInitializer(file=f), name=name)
        return L.Weights(initializer=init or L.NormalInitializer(mean=0.0, standard_deviation=0.02), name=name)

    def linear(self, x, stem: str, size: int, name: str):
        ws = [self.get(stem + ".weight"), self.get(stem + ".bias", L.ConstantInitializer(value=0.0))]
        return L.ChannelwiseFullyConnected(x, weights=ws, output_channel_dims=[size], bias=True, name=name)

    def layer_norm(self, x, stem: str, eps: float, name: str):
        ws = [self.get(stem + ".weight", L.ConstantInitializer(value=1.0)),
              self.get(stem + ".bias", L.ConstantInitializer(value=0.0))]
        return L.LayerNorm(x, epsilon=eps, scale=True, bias=True, start_dim=-1, weights=ws, name=name)


def position_ids_from_input_ids(input_ids, seq_len: int, padding_idx: int):
    """Positions count non-padding tokens from ``padding_idx + 1``; padding keeps ``padding_idx``."""
    pad = L.Constant(value=float(padding_idx), num_neurons=[seq_len])
    mask = L.NotEqual(input_ids, pad)
    inc = Cumsum(L.Reshape(mask, dims=[1, seq_len]), [1, seq_len], axis=1)
    inc = L.Multiply(L.Reshape(inc, dims=[seq_len]), mask)
    return L.Add(inc, pad)


class RobertaLayer(Module):
    def __init__(self, cfg: RobertaConfig, seq_len: int, params: _Params, name: str):
        super().__init__()
        if cfg.hidden_size % cfg.num_attention_heads:
            raise ValueError("hidden_size must be a multiple of num_attention_heads")
        self.cfg, self.S, self.p, self.name = cfg, seq_len, params, name

    def forward(self, x, additive_mask=None):
        c, S, n = self.cfg, self.S, self.name
        H, D = c.num_attention_heads, c.hidden_size // c.num_attention_heads

        def heads(t, tag):
            t = L.Reshape(t, dims=[S, H, D], name=f"{n}.attention.self.{tag}_reshape")
            return L.TensorPermute(t, axes=[1, 0, 2], name=f"{n}.attention.self.{tag}_heads")

        q = heads(self.p.linear(x, f"{n}.attention.self.query", c.hidden_size, f"{n}.attention.self.query"), "q")
        k = heads(self.p.linear(x, f"{n}.attention.self.key", c.hidden_size, f"{n}.attention.self.key"), "k")
        v = heads(self.p.linear(x, f"{n}.attention.self.value", c.hidden_size, f"{n}.attention.self.value"), "v")
        scores = L.Scale(L.MatMul(q, k, transpose_b=True, name=f"{n}.attention.self.scores"),
                         constant=1.0 / math.sqrt(D))
        if additive_mask is not None:
            scores = L.Add(scores, additive_mask, name=f"{n}.attention.self.masked")
        probs = L.ChannelwiseSoftmax(scores, dim=-1, single_dim_mode=True, name=f"{n}.attention.self.softmax")
        if c.attention_probs_dropout_prob > 0:
            probs = L.Dropout(probs, keep_prob=1 - c.attention_probs_dropout_prob)
        ctx = L.TensorPermute(L.MatMul(probs, v, name=f"{n}.attention.self.context"), axes=[1, 0, 2])
        ctx = L.Reshape(ctx, dims=[S, c.hidden_size])
        a = self.p.linear(ctx, f"{n}.attention.output.dense", c.hidden_size, f"{n}.attention.output.dense")
        if c.hidden_dropout_prob > 0:
            a = L.Dropout(a, keep_prob=1 - c.hidden_dropout_prob)
        a = self.p.layer_norm(L.Add(a, x), f"{n}.attention.output.LayerNorm", c.layer_norm_eps,
                              f"{n}.attention.output.LayerNorm")
        h = self.p.linear(a, f"{n}.intermediate.dense", c.intermediate_size, f"{n}.intermediate.dense")
        h = L.Gelu(h, name=f"{n}.intermediate.gelu") if c.hidden_act == "gelu" else L.Relu(h)
        h = self.p.linear(h, f"{n}.output.dense", c.hidden_size, f"{n}.output.dense")
        if c.hidden_dropout_prob > 0:
            h = L.Dropout(h, keep_prob=1 - c.hidden_dropout_prob)
        return self.p.layer_norm(L.Add(h, a), f"{n}.output.LayerNorm", c.layer_norm_eps, f"{n}.output.LayerNorm")


class RoBERTa(Module):
    """``forward(input_ids, token_type_ids=None, attention_mask=None)`` returns the last hidden
    states ``[seq, hidden]`` and, with ``add_pooling_layer``, tanh(dense(first token))."""

    def __init__(self, config: RobertaConfig, seq_len: int, add_pooling_layer: bool = True,
                 load_weights: Union[bool, str, None] = False):
        super().__init__()
        if seq_len + config.pad_token_id + 1 > config.max_position_embeddings:
            raise ValueError("sequence longer than the position table")
        self.cfg, self.S, self.pool = config, seq_len, add_pooling_layer
        self.p = _Params(load_weights)
        self.layers = [RobertaLayer(config, seq_len, self.p, f"encoder.layer.{i}")
                       for i in range(config.num_hidden_layers)]

    def embeddings(self, input_ids, token_type_ids=None):
        c, S, p = self.cfg, self.S, self.p
        pos = position_ids_from_input_ids(input_ids, S, c.pad_token_id)
        if token_type_ids is None:
            token_type_ids = L.Constant(value=0.0, num_neurons=[S])
        e = L.Embedding(input_ids, num_embeddings=c.vocab_size, embedding_dim=c.hidden_size,
                        padding_idx=c.pad_token_id, weights=p.get("embeddings.word_embeddings.weight"),
                        name="embeddings.word_embeddings")
        t = L.Embedding(token_type_ids, num_embeddings=c.type_vocab_size, embedding_dim=c.hidden_size,
                        weights=p.get("embeddings.token_type_embeddings.weight"),
                        name="embeddings.token_type_embeddings")
        e = L.Add(e, t)
        if c.position_embedding_type == "absolute":
            pe = L.Embedding(pos, num_embeddings=c.max_position_embeddings, embedding_dim=c.hidden_size,
                             padding_idx=c.pad_token_id, weights=p.get("embeddings.position_embeddings.weight"),
                             name="embeddings.position_embeddings")
            e = L.Add(e, pe)
        e = p.layer_norm(e, "embeddings.LayerNorm", c.layer_norm_eps, "embeddings.LayerNorm")
        if c.hidden_dropout_prob > 0:
            e = L.Dropout(e, keep_prob=1 - c.hidden_dropout_prob)
        return e

    def extend_attention_mask(self, attention_mask):
        """[seq] of 1 (attend) / 0 (ignore) -> additive [1, seq, seq] mask over the key axis."""
        S = self.S
        m = L.AddConstant(L.Scale(attention_mask, constant=10000.0), constant=-10000.0)     # 0 or -1e4
        return L.Tessellate(L.Reshape(m, dims=[1, 1, S]), dims=[self.cfg.num_attention_heads, S, S])

    def forward(self, input_ids, token_type_ids=None, attention_mask=None):
        x = self.embeddings(input_ids, token_type_ids)
        mask = self.extend_attention_mask(attention_mask) if attention_mask is not None else None
        for layer in self.layers:
            x = layer(x, mask)
        if not self.pool:
            return x
        first = L.Reshape(L.Identity(L.Slice(x, axis=0, slice_points=[0, 1])), dims=[1, self.cfg.hidden_size])
        pooled = L.Tanh(self.p.linear(first, "pooler.dense", self.cfg.hidden_size, "pooler.dense"))
        return x, L.Reshape(pooled, dims=[self.cfg.hidden_size], name="pooler.output")
