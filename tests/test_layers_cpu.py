"""Layer semantics on CPU: every case builds a one-layer graph through the front end, runs it
with lbann.evaluate and compares with the same operation written in PyTorch (fp32)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import lbann_b200 as lbann
from lbann_b200.utils import options as opts

X = np.random.RandomState(0).randn(4, 3, 6, 8).astype(np.float32)
T = torch.from_numpy(X)


def _inp(dims=(3, 6, 8)):
    return lbann.Reshape(lbann.Input(data_field="samples"), dims=list(dims))


UNARY = [
    ("Relu", lambda x: lbann.Relu(x), torch.relu),
    ("LeakyRelu", lambda x: lbann.LeakyRelu(x, negative_slope=0.2), lambda t: F.leaky_relu(t, 0.2)),
    ("Elu", lambda x: lbann.Elu(x, alpha=0.7), lambda t: F.elu(t, 0.7)),
    ("Sigmoid", lambda x: lbann.Sigmoid(x), torch.sigmoid),
    ("Tanh", lambda x: lbann.Tanh(x), torch.tanh),
    ("Softplus", lambda x: lbann.Softplus(x), F.softplus),
    ("Softsign", lambda x: lbann.Softsign(x), F.softsign),
    ("Gelu", lambda x: lbann.Gelu(x), F.gelu),
    ("Selu", lambda x: lbann.Selu(x), F.selu),
    ("Exp", lambda x: lbann.Exp(x), torch.exp),
    ("Abs", lambda x: lbann.Abs(x), torch.abs),
    ("Square", lambda x: lbann.Square(x), torch.square),
    ("Negative", lambda x: lbann.Negative(x), torch.neg),
    ("Sin", lambda x: lbann.Sin(x), torch.sin),
    ("Cos", lambda x: lbann.Cos(x), torch.cos),
    ("Floor", lambda x: lbann.Floor(x), torch.floor),
    ("Sign", lambda x: lbann.Sign(x), torch.sign),
    ("Scale", lambda x: lbann.Scale(x, constant=2.5), lambda t: 2.5 * t),
    ("AddConstant", lambda x: lbann.AddConstant(x, constant=-1.5), lambda t: t - 1.5),
    ("Clamp", lambda x: lbann.Clamp(x, min=-0.5, max=0.25), lambda t: t.clamp(-0.5, 0.25)),
    ("Softmax", lambda x: lbann.Softmax(x), lambda t: torch.softmax(t.reshape(4, -1), 1).reshape(t.shape)),
    ("LogSoftmax", lambda x: lbann.LogSoftmax(x),
     lambda t: torch.log_softmax(t.reshape(4, -1), 1).reshape(t.shape)),
    ("SoftmaxChannel", lambda x: lbann.Softmax(x, softmax_mode="channel"), lambda t: torch.softmax(t, 1)),
    ("ChannelwiseSoftmax", lambda x: lbann.ChannelwiseSoftmax(x),
     lambda t: torch.softmax(t.reshape(4, 3, -1), 2).reshape(t.shape)),
    ("ChannelwiseMean", lambda x: lbann.ChannelwiseMean(x), lambda t: t.mean((2, 3))),
    ("Reduction_sum", lambda x: lbann.Reduction(x, mode="sum"), lambda t: t.reshape(4, -1).sum(1, keepdim=True)),
    ("Reduction_mean", lambda x: lbann.Reduction(x, mode="mean"),
     lambda t: t.reshape(4, -1).mean(1, keepdim=True)),
    ("TensorPermute", lambda x: lbann.TensorPermute(x, axes=[2, 0, 1]), lambda t: t.permute(0, 3, 1, 2)),
    ("Pooling_max", lambda x: lbann.Pooling(x, num_dims=2, has_vectors=False, pool_dims_i=2, pool_pads_i=0,
                                            pool_strides_i=2, pool_mode="max"), lambda t: F.max_pool2d(t, 2)),
    ("Pooling_avg", lambda x: lbann.Pooling(x, num_dims=2, has_vectors=False, pool_dims_i=3, pool_pads_i=1,
                                            pool_strides_i=2, pool_mode="average"),
     lambda t: F.avg_pool2d(t, 3, 2, 1)),
    ("Identity", lambda x: lbann.Identity(x), lambda t: t),
    ("L2Norm2", lambda x: lbann.L2Norm2(x), lambda t: (t * t).reshape(4, -1).sum(1, keepdim=True)),
    ("L1Norm", lambda x: lbann.L1Norm(x), lambda t: t.abs().reshape(4, -1).sum(1, keepdim=True)),
    ("InstanceNorm", lambda x: lbann.InstanceNorm(x, epsilon=1e-5), lambda t: F.instance_norm(t, eps=1e-5)),
    ("LayerNorm", lambda x: lbann.LayerNorm(x, epsilon=1e-5), lambda t: F.layer_norm(t, t.shape[1:], eps=1e-5)),
    ("Crop", None, None),
]


@pytest.mark.parametrize("name,build,ref", [c for c in UNARY if c[1] is not None], ids=lambda v: v if isinstance(v, str) else "")
def test_unary_layer(name, build, ref):
    opts.reset().set("disable_cuda", True)
    out = lbann.evaluate(build(_inp()), X.reshape(4, -1))
    want = ref(T).numpy()
    np.testing.assert_allclose(out.reshape(want.shape), want, rtol=2e-4, atol=2e-5)


BINARY = [
    ("Add", lbann.Add, torch.add), ("Subtract", lbann.Subtract, torch.sub),
    ("Multiply", lbann.Multiply, torch.mul), ("Max", lbann.Max, torch.maximum),
    ("Min", lbann.Min, torch.minimum),
    ("SquaredDifference", lbann.SquaredDifference, lambda a, b: (a - b) ** 2),
    ("Less", lbann.Less, lambda a, b: (a < b).float()),
    ("GreaterEqual", lbann.GreaterEqual, lambda a, b: (a >= b).float()),
]


@pytest.mark.parametrize("name,cls,ref", BINARY, ids=lambda v: v if isinstance(v, str) else "")
def test_binary_layer(name, cls, ref):
    opts.reset().set("disable_cuda", True)
    x = _inp()
    y = lbann.Tanh(x)
    out = lbann.evaluate(cls(x, y), X.reshape(4, -1))
    want = ref(T, torch.tanh(T)).numpy()
    np.testing.assert_allclose(out.reshape(want.shape), want, rtol=2e-4, atol=2e-5)


def test_slice_concat_sum_split():
    opts.reset().set("disable_cuda", True)
    x = _inp()
    s = lbann.Slice(x, axis=0, slice_points=[0, 1, 3])
    a, b = lbann.Identity(s), lbann.Identity(s)
    cat = lbann.Concatenation([b, a], axis=0)
    tot = lbann.Sum(cat, x)
    out = lbann.evaluate(tot, X.reshape(4, -1))
    want = (torch.cat([T[:, 1:3], T[:, 0:1]], 1) + T).numpy()
    np.testing.assert_allclose(out.reshape(want.shape), want, rtol=1e-5)


def test_convolution_deconvolution_fc_embedding_match_torch():
    opts.reset().set("disable_cuda", True)
    rs = np.random.RandomState(1)
    wk = rs.randn(5, 3, 3, 3).astype(np.float32) * 0.2
    wd = rs.randn(5, 2, 2, 2).astype(np.float32) * 0.2
    x = _inp()
    conv = lbann.Convolution(x, num_dims=2, out_channels=5, kernel_size=3, padding=1, stride=2, has_bias=False,
                             weights=[lbann.Weights(initializer=lbann.ValueInitializer(values=wk.reshape(-1).tolist()))])
    dec = lbann.Deconvolution(conv, num_dims=2, out_channels=2, kernel_size=2, stride=2, padding=0, has_bias=False,
                              weights=[lbann.Weights(initializer=lbann.ValueInitializer(values=wd.reshape(-1).tolist()))])
    got_c, got_d = lbann.evaluate([conv, dec], X.reshape(4, -1), outputs=[conv.name, dec.name])
    ref_c = F.conv2d(T, torch.from_numpy(wk), None, 2, 1)
    ref_d = F.conv_transpose2d(ref_c, torch.from_numpy(wd), None, 2, 0)
    np.testing.assert_allclose(got_c, ref_c.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(got_d, ref_d.numpy(), rtol=1e-4, atol=1e-5)
    # embedding: indices in, rows of the table out
    table = rs.randn(7, 4).astype(np.float32)
    idx = np.array([[0, 3, 6], [2, 2, 5]], dtype=np.float32)
    emb = lbann.Embedding(lbann.Input(data_field="samples"), num_embeddings=7, embedding_dim=4,
                          weights=lbann.Weights(initializer=lbann.ValueInitializer(values=table.reshape(-1).tolist())))
    got = lbann.evaluate(emb, idx)
    np.testing.assert_allclose(got, table[idx.astype(int)], rtol=1e-6)


def test_every_frontend_layer_class_exports_a_message():
    """The generated front end covers the whole layer schema: each class can be
    instantiated without arguments and produces a Layer message of its own type."""
    from lbann_b200.proto import lbann_pb2
    oneof = lbann_pb2.Layer.DESCRIPTOR.oneofs_by_name["layer_type"]
    missing = []
    for f in oneof.fields:
        cls_name = f.message_type.name
        cls = getattr(lbann, cls_name, None)
        if cls is None:
            missing.append(cls_name)
            continue
        msg = cls().export_proto()
        assert msg.WhichOneof("layer_type") == f.name, cls_name
    assert not missing, missing


def test_batch_norm_counts_the_whole_mini_batch_when_shares_differ():
    """Whole-trainer statistics: the count is global mini-batch x entries per sample, not this
    rank's entries x ranks (a last mini-batch of 3 samples leaves 2 + 1 on two ranks)."""
    from types import SimpleNamespace
    from lbann_b200.exec.layers_core import BatchNormalization
    bn = BatchNormalization.__new__(BatchNormalization)
    bn.in_dims = [(8, 4, 4)]
    par = SimpleNamespace(world_size=2, tp_size=1)
    bn.model = SimpleNamespace(parallel=par, subgrid=None, _global_mb=3, _global_mb_given=True)
    two, one = torch.zeros(2, 8, 4, 4), torch.zeros(1, 8, 4, 4)
    assert bn.exact_count_scale(two, 2.0) == 3 * 16 / (2 * 16)
    assert bn.exact_count_scale(one, 2.0) == 3.0
    bn.model._global_mb = 4                          # equal shares: exactly the number of ranks
    assert bn.exact_count_scale(two, 2.0) == 2.0
    bn.model._global_mb_given = False                # size not passed by the caller: unchanged
    assert bn.exact_count_scale(one, 2.0) == 2.0
    bn.model._global_mb_given = True
    assert bn.exact_count_scale(one, 4.0) == 4.0     # statistics of a sub-group of ranks: unchanged
    bn.in_dims = [(8,)]
    assert bn.exact_count_scale(torch.zeros(1, 8), 2.0) == 4.0
