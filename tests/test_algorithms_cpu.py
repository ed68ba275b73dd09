"""lbann.evaluate, K-FAC and prototext round trips on CPU."""
import math

import numpy as np
import pytest
import torch

import lbann_b200 as lbann
from lbann_b200.exec.trainer import ExecTrainer
from lbann_b200.utils import options as opts
from test_models_cpu import _reader


def test_evaluate_returns_forward_outputs():
    opts.reset().set("disable_cuda", True)
    x = lbann.Input(data_field="samples")
    w = lbann.Weights(initializer=lbann.ValueInitializer(values=[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]),
                      name="w")
    y = lbann.FullyConnected(x, num_neurons=2, has_bias=False, weights=[w], name="fc")
    z = lbann.Relu(y, name="out")
    inp = np.array([[1.0, 0.0, -1.0], [0.5, 0.5, 0.5]], dtype=np.float32)
    out = lbann.evaluate(z, inp)
    W = np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], dtype=np.float32)
    ref = np.maximum(inp @ W.T, 0)
    # the value list fills the matrix in column-major order like the reference
    ref_cm = np.maximum(inp @ W.reshape(3, 2), 0)
    assert np.allclose(out, ref, atol=1e-5) or np.allclose(out, ref_cm, atol=1e-5), out
    both = lbann.evaluate(z, inp, outputs=["fc", "out"])
    assert isinstance(both, tuple) and both[0].shape == (2, 2)
    assert np.allclose(np.maximum(both[0], 0), both[1])


def _mlp():
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    h = lbann.Tanh(lbann.FullyConnected(x, num_neurons=16, has_bias=True, name="fc1"))
    y = lbann.FullyConnected(h, num_neurons=3, has_bias=True, name="fc2")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    return lbann.Model(3, layers=list(lbann.traverse_layer_graph([x, t])),
                       objective_function=lbann.ObjectiveFunction([loss]))


def _fit(algo, epochs=3, cuda=False):
    o = opts.reset()
    if not cuda:
        o.set("disable_cuda", True)
    torch.manual_seed(0)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=16, random_seed=9, training_algo=algo), model=_mlp(),
        data_reader=_reader(64, [8], "normal", response_dims=[3]),
        optimizer=lbann.SGD(learn_rate=0.05, momentum=0.0))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tr.train(m, num_epochs=epochs)
    obj, _, _ = m.reduce_statistics("training")
    tr.shutdown()
    return obj


def test_kfac_preconditioning_speeds_up_sgd():
    sgd = lbann.BatchedIterativeOptimizer("sgd", epoch_count=3)
    kfac = lbann.KFAC("kfac", sgd, damping_act="1e-2", damping_err="1e-2", kronecker_decay=0.9,
                      update_intervals="1", compute_interval=1)
    plain = _fit(sgd)
    second = _fit(kfac)
    assert math.isfinite(second) and second < plain, (plain, second)


def test_prototext_round_trip(tmp_path):
    from google.protobuf import text_format
    from lbann_b200.proto import lbann_pb2
    model = _mlp()
    msg = lbann.proto.serialize.save_prototext(
        str(tmp_path / "exp.prototext"), trainer=lbann.Trainer(mini_batch_size=4), model=model,
        data_reader=_reader(8, [8], "normal", response_dims=[3]), optimizer=lbann.Adam(learn_rate=1e-3))
    back = lbann_pb2.LbannPB()
    text_format.Parse(open(tmp_path / "exp.prototext").read(), back)
    assert back == msg
    assert [l.name for l in back.model.layer if l.HasField("fully_connected")] == ["fc1", "fc2"]


def test_torch_module_lowering_matches_pytorch():
    import torch.nn as nn
    import lbann_b200.torch as lt
    opts.reset().set("disable_cuda", True)
    torch.manual_seed(0)
    net = nn.Sequential(nn.Conv2d(2, 4, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Flatten(),
                        nn.Linear(4 * 4 * 4, 5), nn.Tanh())
    x = torch.randn(3, 2, 8, 8)
    outs = lt.compile(net, input=x)
    got = lbann.evaluate(outs[0], x.numpy())
    torch.testing.assert_close(torch.from_numpy(got), net(x).detach(), rtol=1e-4, atol=1e-5)
