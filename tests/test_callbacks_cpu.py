"""Checkpoint / restart, weight dumps, learning-rate schedules and early termination through
the callback interface, on the LeNet CPU configuration."""
import os

import numpy as np
import pytest
import torch

import lbann_b200 as lbann
from lbann_b200.exec.trainer import ExecTrainer
from lbann_b200.utils import options as opts
from test_lenet_cpu import build_lenet, make_reader


def _experiment(callbacks, epochs, lr=0.01):
    images, labels, loss, acc = build_lenet()
    model = lbann.Model(epochs, layers=[images, labels], objective_function=loss,
                        metrics=[lbann.Metric(acc, name="accuracy", unit="%")], callbacks=callbacks)
    return lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=64, random_seed=7), model=model,
        data_reader=make_reader(128), optimizer=lbann.SGD(learn_rate=lr, momentum=0.9))


def _run(exp, epochs):
    opts.reset().set("disable_cuda", True)
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tr.train(m, num_epochs=epochs)
    weights = {w.name: w.values.detach().clone() for w in m.weights}
    state = (m.ctx.epoch, m.ctx.step)
    lrs = {w.name: w.slot.hp.get("learn_rate") for w in m.weights if w.has_optimizer()}
    tr.shutdown()
    return weights, state, lrs


def test_checkpoint_restart_reproduces_uninterrupted_run(tmp_path):
    ck = str(tmp_path / "ckpt")
    # uninterrupted: 4 epochs
    ref, ref_state, _ = _run(_experiment([], 4), 4)
    # 2 epochs with a checkpoint at the end, then a fresh process state resumes to 4
    _run(_experiment([lbann.CallbackCheckpoint(checkpoint_dir=ck, checkpoint_epochs=1)], 2), 2)
    tdir = os.path.join(ck, "trainer")
    assert os.path.isfile(os.path.join(tdir, "last.shared.checkpoint")) or os.listdir(ck), os.listdir(ck)
    got, state, _ = _run(_experiment([lbann.CallbackCheckpoint(checkpoint_dir=ck, checkpoint_epochs=1)], 4), 4)
    assert state == ref_state
    for k, v in ref.items():
        torch.testing.assert_close(got[k], v, rtol=1e-5, atol=1e-6, msg=k)


def test_dump_weights_and_step_learning_rate(tmp_path):
    d = str(tmp_path / "w")
    cbs = [lbann.CallbackDumpWeights(directory=d, epoch_interval=1, format="npy"),
           lbann.CallbackStepLearningRate(step=1, amt=0.5)]
    _, _, lrs = _run(_experiment(cbs, 2, lr=0.02), 2)
    files = [f for _, _, fs in os.walk(d) for f in fs]
    assert any(f.endswith(".npy") for f in files), files
    assert all(abs(v - 0.02 * 0.25) < 1e-9 for v in lrs.values()), lrs


def test_early_stopping_ends_training(tmp_path):
    # patience 0 on a metric that cannot improve every epoch forever: stops before 30 epochs
    cbs = [lbann.CallbackEarlyStopping(patience=1)]
    exp = _experiment(cbs, 30)
    exp.data_reader.reader[1].role = "validate"
    _, (epoch, _), _ = _run(exp, 30)
    assert epoch < 30


def test_export_onnx_writes_a_model_that_a_numpy_interpreter_reproduces(tmp_path):
    """The export callback writes a binary ONNX ModelProto.  It is parsed back and run by a
    small NumPy interpreter (Conv, MaxPool, Flatten, Gemm, Relu, LeakyRelu, Concat, Reshape,
    Softmax): same outputs as the framework's own forward pass."""
    import numpy as np
    import torch
    import torch.nn.functional as F
    import lbann_b200 as lbann
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.io import onnx_proto as op
    from lbann_b200.utils import options as opts
    opts.reset().set("disable_cuda", True)
    x = lbann.Input(data_field="samples", name="img")
    c = lbann.Convolution(x, num_dims=2, out_channels=3, kernel_size=[3, 3], padding=[1, 1], stride=[1, 1],
                          has_bias=True, name="conv")
    a = lbann.LeakyRelu(c, negative_slope=0.1, name="lrelu")
    p = lbann.Pooling(a, num_dims=2, has_vectors=False, pool_dims_i=2, pool_pads_i=0, pool_strides_i=2,
                      pool_mode="max", name="pool")
    f1 = lbann.Relu(lbann.FullyConnected(p, num_neurons=5, has_bias=True, name="fc1"), name="relu1")
    f2 = lbann.FullyConnected(lbann.Reshape(p, dims=[27], name="flat"), num_neurons=4, has_bias=False, name="fc2")
    y = lbann.Softmax(lbann.Concatenation([f1, f2], axis=0, name="cat"), name="probs")
    onnx_file, text_file = str(tmp_path / "m.onnx"), str(tmp_path / "m.txt")
    model = lbann.Model(0, layers=list(lbann.traverse_layer_graph(x)),
                        callbacks=[lbann.CallbackExportOnnx(output_filename=onnx_file, debug_string_filename=text_file)])
    data = np.random.RandomState(0).randn(4, 2, 6, 6).astype(np.float32)
    from lbann_b200.data.readers import ArrayReader
    exp = lbann.proto.serialize.build_experiment(trainer=lbann.Trainer(mini_batch_size=4), model=model,
                                                 data_reader=None, optimizer=lbann.NoOptimizer())
    tr = ExecTrainer(exp, readers={"train": ArrayReader({"samples": data}, role="train")})
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    with torch.no_grad():
        m.forward_prop(b.tensors, "training", b.global_size, 0)
    want = m.acts["probs"][0].float().numpy()
    for cb in m.callbacks:
        cb.on_train_end(m)
    tr.shutdown()

    mp = op.ModelProto()
    mp.ParseFromString(open(onnx_file, "rb").read())
    assert mp.opset_import[0].version == 11 and mp.producer_name == "lbann_b200"
    assert [i.name for i in mp.graph.input] == ["img_out0"] and [o.name for o in mp.graph.output] == ["probs_out0"]
    assert [d.dim_param or d.dim_value for d in mp.graph.input[0].type.tensor_type.shape.dim] == ["batch", 2, 6, 6]
    assert 'op_type: "Conv"' in open(text_file).read()
    env = {"img_out0": data}
    for t in mp.graph.initializer:
        dt = np.int64 if t.data_type == op.INT64 else np.float32
        env[t.name] = np.frombuffer(t.raw_data, dtype=dt).reshape(tuple(t.dims)).copy()
    attr = lambda n: {a.name: (list(a.ints) if a.type == op.ATTR_INTS else a.i if a.type == op.ATTR_INT else a.f)
                      for a in n.attribute}                                                     # noqa: E731
    for n in mp.graph.node:
        i, at = [env[k] for k in n.input], attr(n)
        if n.op_type == "Conv":
            nd = len(at["kernel_shape"])
            assert at["pads"] == [1] * (2 * nd) and at["group"] == 1
            r = F.conv2d(torch.from_numpy(i[0]), torch.from_numpy(i[1]), torch.from_numpy(i[2]),
                         at["strides"], at["pads"][:nd], at["dilations"]).numpy()
        elif n.op_type == "LeakyRelu":
            r = np.where(i[0] > 0, i[0], at["alpha"] * i[0])
        elif n.op_type == "Relu":
            r = np.maximum(i[0], 0)
        elif n.op_type == "MaxPool":
            r = F.max_pool2d(torch.from_numpy(i[0]), at["kernel_shape"], at["strides"], at["pads"][:2]).numpy()
        elif n.op_type == "Flatten":
            r = i[0].reshape(i[0].shape[0], -1)
        elif n.op_type == "Gemm":
            r = i[0] @ (i[1].T if at.get("transB") else i[1]) + (i[2] if len(i) > 2 else 0.0)
        elif n.op_type == "Reshape":
            shape = [i[0].shape[k] if v == 0 else int(v) for k, v in enumerate(i[1])]
            r = i[0].reshape(shape)
        elif n.op_type == "Concat":
            r = np.concatenate(i, axis=at["axis"])
        elif n.op_type == "Softmax":
            z = i[0].reshape(i[0].shape[0], -1)
            e = np.exp(z - z.max(1, keepdims=True))
            r = (e / e.sum(1, keepdims=True)).reshape(i[0].shape)
        elif n.op_type == "Identity":
            r = i[0]
        else:
            raise AssertionError(f"unexpected node {n.op_type} ({n.domain})")
        env[n.output[0]] = r
    np.testing.assert_allclose(env["probs_out0"].reshape(want.shape), want, rtol=1e-5, atol=1e-6)
