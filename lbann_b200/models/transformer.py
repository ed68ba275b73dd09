"""Transformer encoder / decoder stacks and a GPT-style decoder-only language model.

Layer structure and weight names follow the reference's ``lbann.models.Transformer``
(python/lbann/models/transformer.py:21-675): post- or pre-LayerNorm residual blocks of
multi-head attention and a two-layer feed-forward network on ``[sequence, embed]`` tensors.
``GPT`` adds what the decoder-only benchmark needs: token + learned position embeddings,
causal mask, tied or separate LM head and the per-token cross-entropy.
"""
from __future__ import annotations

import numpy as np

from ..frontend import core as L
from ..modules.base import ChannelwiseFullyConnectedModule, Module
from ..modules.transformer import (LearnedInputEncoding, MultiheadAttention, PositionalEncoding,
                                   RotaryPositionalEmbedding)


class LayerNorm(Module):
    """Layer normalisation over the embedding dimension with learned scale and bias."""

    global_count = 0

    def __init__(self, normalized_shape, name=None, builtin=True):
        super().__init__()
        LayerNorm.global_count += 1
        self.normalized_shape = normalized_shape
        self.name = name or f"layernorm{LayerNorm.global_count}"
        self.instance = 0
        self.weight = L.Weights(initializer=L.ConstantInitializer(value=1), name=f"{self.name}_weight")
        self.bias = L.Weights(initializer=L.ConstantInitializer(value=0), name=f"{self.name}_bias")

    def forward(self, x):
        self.instance += 1
        return L.LayerNorm(x, scale=True, bias=True, start_dim=-1, weights=[self.weight, self.bias],
                           name=f"{self.name}_instance{self.instance}")


class _FeedForward(Module):
    def __init__(self, embed_dim, ff_dim, dropout, activation, name):
        super().__init__()
        self.dropout, self.activation, self.name = dropout, activation, name
        self.fc1 = ChannelwiseFullyConnectedModule(ff_dim, weights=[
            L.Weights(initializer=L.GlorotNormalInitializer(), name=f"{name}_fc1_matrix"),
            L.Weights(initializer=L.ConstantInitializer(value=0), name=f"{name}_fc1_bias")],
            name=f"{name}_fc1")
        self.fc2 = ChannelwiseFullyConnectedModule(embed_dim, weights=[
            L.Weights(initializer=L.GlorotNormalInitializer(), name=f"{name}_fc2_matrix"),
            L.Weights(initializer=L.ConstantInitializer(value=0), name=f"{name}_fc2_bias")],
            name=f"{name}_fc2")
        self.instance = 0

    def forward(self, x):
        self.instance += 1
        n = f"{self.name}_ffn{self.instance}"
        y = self.activation(self.fc1(x), name=f"{n}_act")
        if self.dropout > 0:
            y = L.Dropout(y, keep_prob=1 - self.dropout, name=f"{n}_drop1")
        y = self.fc2(y)
        if self.dropout > 0:
            y = L.Dropout(y, keep_prob=1 - self.dropout, name=f"{n}_drop2")
        return y


class TransformerEncoderLayer(Module):
    global_count = 0

    def __init__(self, embed_dim=512, num_heads=8, feedforward_dim=2048, dropout=0.1,
                 attn_dropout=0.0, pre_layernorm=False, activation=L.Relu, name=None,
                 attention_bias=None, positional_encoding=None, branches=0):
        super().__init__()
        TransformerEncoderLayer.global_count += 1
        self.name = name or f"transformerencoderlayer{TransformerEncoderLayer.global_count}"
        self.embed_dim, self.dropout, self.pre_ln = embed_dim, dropout, pre_layernorm
        self.attention = MultiheadAttention(embed_dim, num_heads, self_attention=True,
                                            dropout=attn_dropout, bias=attention_bias,
                                            positional_encoding=positional_encoding,
                                            subgraph_branches=branches,
                                            name=f"{self.name}_attention")
        self.norm1 = LayerNorm(embed_dim, name=f"{self.name}_norm1")
        self.norm2 = LayerNorm(embed_dim, name=f"{self.name}_norm2")
        self.ffn = _FeedForward(embed_dim, feedforward_dim, dropout, activation, self.name)
        self.instance = 0

    def forward(self, x, mask=None):
        self.instance += 1
        n = f"{self.name}_instance{self.instance}"
        h = self.norm1(x) if self.pre_ln else x
        a = self.attention(h, h, h, mask=mask)
        if self.dropout > 0:
            a = L.Dropout(a, keep_prob=1 - self.dropout, name=f"{n}_drop1")
        x = L.Sum(x, a, name=f"{n}_sum1")
        if not self.pre_ln:
            x = self.norm1(x)
        h = self.norm2(x) if self.pre_ln else x
        x = L.Sum(x, self.ffn(h), name=f"{n}_sum2")
        if not self.pre_ln:
            x = self.norm2(x)
        return x


class TransformerDecoderLayer(Module):
    global_count = 0

    def __init__(self, embed_dim=512, num_heads=8, feedforward_dim=2048, dropout=0.1,
                 attn_dropout=0.0, pre_layernorm=False, activation=L.Relu, name=None,
                 attention_bias=None, positional_encoding=None, branches=0):
        super().__init__()
        TransformerDecoderLayer.global_count += 1
        self.name = name or f"transformerdecoderlayer{TransformerDecoderLayer.global_count}"
        self.embed_dim, self.dropout, self.pre_ln = embed_dim, dropout, pre_layernorm
        self.attention1 = MultiheadAttention(embed_dim, num_heads, self_attention=True,
                                             dropout=attn_dropout, bias=attention_bias,
                                             positional_encoding=positional_encoding,
                                             subgraph_branches=branches,
                                             name=f"{self.name}_attention1")
        self.attention2 = MultiheadAttention(embed_dim, num_heads, dropout=attn_dropout,
                                             positional_encoding=positional_encoding,
                                             subgraph_branches=branches,
                                             name=f"{self.name}_attention2")
        self.norm1 = LayerNorm(embed_dim, name=f"{self.name}_norm1")
        self.norm2 = LayerNorm(embed_dim, name=f"{self.name}_norm2")
        self.norm3 = LayerNorm(embed_dim, name=f"{self.name}_norm3")
        self.ffn = _FeedForward(embed_dim, feedforward_dim, dropout, activation, self.name)
        self.instance = 0

    def forward(self, x, memory=None, src_mask=None, tgt_mask=None):
        self.instance += 1
        n = f"{self.name}_instance{self.instance}"

        def block(x, norm, fn, tag):
            h = norm(x) if self.pre_ln else x
            y = fn(h)
            if self.dropout > 0:
                y = L.Dropout(y, keep_prob=1 - self.dropout, name=f"{n}_drop{tag}")
            x = L.Sum(x, y, name=f"{n}_sum{tag}")
            return x if self.pre_ln else norm(x)

        x = block(x, self.norm1, lambda h: self.attention1(h, h, h, mask=tgt_mask), 1)
        if memory is not None:
            x = block(x, self.norm2, lambda h: self.attention2(h, memory, memory, mask=src_mask), 2)
        return block(x, self.norm3, self.ffn, 3)


def causal_mask(seq_len: int, name: str = "causal_mask"):
    """Additive ``[1, S, S]`` mask with -1e9 above the diagonal (constant weights)."""
    m = np.triu(np.full((seq_len, seq_len), -1e9, dtype=np.float32), k=1)
    w = L.Weights(initializer=L.ValueInitializer(values=m.reshape(-1).tolist()),
                  optimizer=L.NoOptimizer(), name=f"{name}_values")
    return L.WeightsLayer(weights=w, dims=[1, seq_len, seq_len], name=name)


class Transformer(Module):
    """Encoder-decoder stack; ``forward(source, target)`` returns the decoder output.
    ``branches`` = B > 0: the attention heads of every layer run on B sub-grids of the trainer
    (sub-graph parallelism; run with ``--num-subgrids B``)."""

    global_count = 0

    def __init__(self, hidden_size=512, num_heads=8, num_encoder_layers=6, num_decoder_layers=6,
                 feedforward_size=None, dropout=0.1, attn_dropout=0.0, pre_layernorm=False,
                 activation=L.Relu, name=None, positional_encoding=None, branches=0):
        super().__init__()
        Transformer.global_count += 1
        self.name = name or f"transformer{Transformer.global_count}"
        self.hidden_size = hidden_size
        ff = feedforward_size or 4 * hidden_size
        kw = dict(embed_dim=hidden_size, num_heads=num_heads, feedforward_dim=ff, dropout=dropout,
                  attn_dropout=attn_dropout, pre_layernorm=pre_layernorm, activation=activation,
                  positional_encoding=positional_encoding, branches=branches)
        self.encoder = [TransformerEncoderLayer(name=f"{self.name}_encoder{i}", **kw)
                        for i in range(num_encoder_layers)]
        self.decoder = [TransformerDecoderLayer(name=f"{self.name}_decoder{i}", **kw)
                        for i in range(num_decoder_layers)]
        self.separate_final_norm = pre_layernorm
        if pre_layernorm:
            self.enc_norm = LayerNorm(hidden_size, name=f"{self.name}_encoder_norm")
            self.dec_norm = LayerNorm(hidden_size, name=f"{self.name}_decoder_norm")

    def forward(self, source, target, target_length=None, cross_attention=True):
        x = source
        for layer in self.encoder:
            x = layer(x)
        memory = self.enc_norm(x) if self.encoder and self.separate_final_norm else x
        if not self.decoder:
            return memory
        mask = causal_mask(target_length, f"{self.name}_mask") if target_length else None
        y = target
        for layer in self.decoder:
            y = layer(y, memory if (cross_attention and self.encoder) else None, tgt_mask=mask)
        return self.dec_norm(y) if self.separate_final_norm else y


class GPT(Module):
    """Decoder-only language model: embeddings + ``num_layers`` pre-LayerNorm blocks +
    final LayerNorm + LM head; ``forward(tokens)`` returns ``[S, vocab]`` logits."""

    def __init__(self, vocab_size=50304, seq_len=2048, d_model=2048, num_heads=16, num_layers=24,
                 ffn_dim=8192, dropout=0.0, tie_embeddings=False, positional_encoding="learned",
                 name="gpt"):
        super().__init__()
        self.name, self.vocab, self.seq_len, self.d_model = name, vocab_size, seq_len, d_model
        if positional_encoding not in ("learned", "sinusoidal", "rope"):
            raise ValueError(f"unknown positional encoding {positional_encoding!r}")
        self.embed_weights = L.Weights(initializer=L.NormalInitializer(standard_deviation=0.02),
                                       name=f"{name}_token_embeddings")
        # learned / sinusoidal encodings act on the embedded input, rotary embedding on every
        # layer's queries and keys (applications/nlp/transformer/modeling.py:132-200)
        layer_enc = None
        if positional_encoding == "learned":
            self.positions = LearnedInputEncoding(d_model, seq_len, dropout=dropout, name=f"{name}_positions")
        elif positional_encoding == "sinusoidal":
            self.positions = PositionalEncoding(d_model, dropout=dropout, name=f"{name}_positions")
        else:
            self.positions = None
            layer_enc = RotaryPositionalEmbedding(d_model // num_heads, seq_len, num_heads, name=f"{name}_rope")
        self.blocks = [TransformerEncoderLayer(embed_dim=d_model, num_heads=num_heads,
                                               feedforward_dim=ffn_dim, dropout=dropout,
                                               pre_layernorm=True, activation=L.Gelu,
                                               positional_encoding=layer_enc,
                                               name=f"{name}_block{i}") for i in range(num_layers)]
        self.final_norm = LayerNorm(d_model, name=f"{name}_final_norm")
        self.tie = tie_embeddings
        self.head = ChannelwiseFullyConnectedModule(
            vocab_size, bias=False, transpose=False,   # the table is [vocab, d_model] = [out, in]
            weights=[self.embed_weights] if tie_embeddings else
            [L.Weights(initializer=L.NormalInitializer(standard_deviation=0.02), name=f"{name}_lm_head")],
            name=f"{name}_head")

    def forward(self, tokens):
        x = L.Embedding(tokens, num_embeddings=self.vocab, embedding_dim=self.d_model,
                        weights=self.embed_weights, name=f"{self.name}_embed")
        if self.positions is not None:
            x = self.positions.apply_input(x, self.seq_len)
        mask = causal_mask(self.seq_len, f"{self.name}_causal")
        for blk in self.blocks:
            x = blk(x, mask=mask)
        return self.head(self.final_norm(x))


def construct_gpt_model(vocab_size=50304, seq_len=2048, d_model=2048, num_heads=16, num_layers=24,
                        ffn_dim=8192, num_epochs=1, callbacks=(), **kw):
    """A complete ``lbann.Model``: tokens ``[S + 1]`` per sample (inputs + next-token labels),
    mean per-token softmax cross-entropy."""
    inp = L.Input(data_field="samples", name="tokens")
    sl = L.Slice(L.Reshape(inp, dims=[seq_len + 1]), axis=0, slice_points=[0, seq_len, seq_len + 1],
                 name="token_slice")
    tokens = L.Identity(sl, name="input_tokens")
    L.Identity(sl, name="last_token")     # keeps the slice's second output connected
    lab = L.Slice(L.Reshape(inp, dims=[seq_len + 1], name="labels_view"), axis=0,
                  slice_points=[0, 1, seq_len + 1], name="label_slice")
    L.Identity(lab, name="first_token")
    labels = L.Identity(lab, name="next_tokens")
    net = GPT(vocab_size, seq_len, d_model, num_heads, num_layers, ffn_dim, **kw)
    logits = net(tokens)                                     # [S, vocab]
    # class dimension first, as the label-index cross-entropy wants it; the permute is a
    # view and softmax + cross-entropy run as one fused kernel on the logits
    probs = L.Softmax(L.TensorPermute(logits, axes=[1, 0], name="logits_t"), softmax_mode="channel",
                      name="token_probs")
    ce = L.CrossEntropy(probs, labels, use_labels=True, name="ce_sum")
    loss = L.Scale(ce, constant=1.0 / seq_len, name="loss")
    layers = list(L.traverse_layer_graph([inp]))
    return L.Model(num_epochs, layers=layers, objective_function=L.ObjectiveFunction([loss]),
                   metrics=[L.Metric(loss, name="loss")], callbacks=list(callbacks))
