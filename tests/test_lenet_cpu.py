"""LeNet-5 on CPU in fp32 through the public front end: trains, objective decreases."""
import io
import contextlib
import re

import lbann_b200 as lbann


def build_lenet(num_labels=10):
    images = lbann.Input(data_field="samples")
    labels = lbann.Input(data_field="labels")
    x = lbann.Convolution(images, num_dims=2, out_channels=6, kernel_size=5, padding=0, stride=1,
                          has_bias=True, name="conv1")
    x = lbann.Relu(x)
    x = lbann.Pooling(x, num_dims=2, pool_dims_i=2, pool_pads_i=0, pool_strides_i=2, pool_mode="max")
    x = lbann.Convolution(x, num_dims=2, out_channels=16, kernel_size=5, has_bias=True, name="conv2")
    x = lbann.Relu(x)
    x = lbann.Pooling(x, num_dims=2, pool_dims_i=2, pool_pads_i=0, pool_strides_i=2, pool_mode="max")
    x = lbann.FullyConnected(x, num_neurons=120, has_bias=True, name="fc1")
    x = lbann.Relu(x)
    x = lbann.FullyConnected(x, num_neurons=84, has_bias=True, name="fc2")
    x = lbann.Relu(x)
    x = lbann.FullyConnected(x, num_neurons=num_labels, has_bias=True, name="fc3")
    probs = lbann.Softmax(x)
    loss = lbann.CrossEntropy(probs, labels)
    acc = lbann.CategoricalAccuracy(probs, labels)
    return images, labels, loss, acc


def make_reader(n=256):
    rd = lbann.reader_pb2.DataReader()
    for role, cnt in (("train", n), ("test", 64)):
        r = rd.reader.add()
        r.name = "synthetic"
        r.role = role
        r.num_samples = cnt
        r.num_labels = 10
        r.synth_dimensions = "1 28 28"
        r.synth_distribution = "uniform"
        r.shuffle = role == "train"
        r.fraction_of_data_to_use = 1.0
    return rd


def test_lenet_trains_on_cpu(tmp_path):
    images, labels, loss, acc = build_lenet()
    model = lbann.Model(3, layers=[images, labels], objective_function=loss,
                        metrics=[lbann.Metric(acc, name="accuracy", unit="%")],
                        callbacks=[lbann.CallbackPrint(), lbann.CallbackTimer()])
    trainer = lbann.Trainer(mini_batch_size=64, random_seed=7)
    opt = lbann.SGD(learn_rate=0.01, momentum=0.9)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        rc = lbann.run(trainer, model, make_reader(), opt, work_dir=str(tmp_path),
                       lbann_args=["--disable_cuda"])
    out = buf.getvalue()
    assert rc == 0
    objs = [float(v) for v in re.findall(r"training epoch \d+ objective function : ([-\d.e+]+)", out)]
    assert len(objs) == 3
    assert objs[-1] < objs[0]
    assert "test objective function" in out
    assert "mini-batch time statistics" in out
    assert (tmp_path / "experiment.prototext").exists()


def test_cuda_graph_option_is_ignored_without_a_gpu():
    """use_cuda_graph on a CPU run: the model decides against capturing and trains step by
    step."""
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.utils import options as opts
    from test_models_cpu import _reader
    o = opts.reset()
    o.set("disable_cuda", True)
    o.set("use_cuda_graph", True)
    x = lbann.Input(data_field="samples")
    y = lbann.FullyConnected(x, num_neurons=3)
    loss = lbann.MeanSquaredError(y, lbann.Input(data_field="responses"))
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=4), model=model,
        data_reader=_reader(8, [5], "normal", response_dims=[3]), optimizer=lbann.SGD(learn_rate=0.05))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    first = float(m.train_step(b.tensors, b.global_size))
    for _ in range(5):
        last = float(m.train_step(b.tensors, b.global_size))
    tr.shutdown()
    opts.reset()
    assert m._graph_mode is False and not m._graphs
    assert last < first


def test_snapshot_and_restore_replay_the_same_steps():
    """``snapshot_state`` / ``restore_state``: weights, Adam moments and step counters go back
    to where they were, so the same mini-batches give the same losses again."""
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.utils import options as opts
    from test_models_cpu import _reader
    o = opts.reset()
    o.set("disable_cuda", True)
    x = lbann.Input(data_field="samples")
    y = lbann.FullyConnected(lbann.Relu(lbann.FullyConnected(x, num_neurons=7)), num_neurons=3)
    loss = lbann.MeanSquaredError(y, lbann.Input(data_field="responses"))
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=4), model=model,
        data_reader=_reader(8, [5], "normal", response_dims=[3]), optimizer=lbann.Adam(learn_rate=0.05))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    snap = m.snapshot_state()
    first = [float(m.train_step(b.tensors, b.global_size)) for _ in range(4)]
    m.restore_state(snap)
    again = [float(m.train_step(b.tensors, b.global_size)) for _ in range(4)]
    tr.shutdown()
    opts.reset()
    assert first[-1] < first[0]
    assert again == first
