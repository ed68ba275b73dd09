"""Front-end helpers: hyper-parameter grid search files and the per-trainer experiment files
of the driver."""
import csv
import os

import lbann_b200 as lbann
from lbann_b200.contrib.hyperparameter import grid_search
from lbann_b200.launcher import make_batch_script


def _experiment(learn_rate, width):
    x = lbann.Input(data_field="samples")
    y = lbann.FullyConnected(lbann.Relu(lbann.FullyConnected(x, num_neurons=width)), num_neurons=4)
    loss = lbann.MeanSquaredError(y, lbann.Input(data_field="responses"))
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x])),
                        objective_function=lbann.ObjectiveFunction([loss]),
                        callbacks=[lbann.CallbackPrint()])
    r = lbann.reader_pb2.Reader(name="synthetic", role="train", num_samples=16, synth_dimensions="8",
                                synth_response_dimensions="4", fraction_of_data_to_use=1.0)
    reader = lbann.reader_pb2.DataReader()
    reader.reader.append(r)
    return model, lbann.SGD(learn_rate=learn_rate), reader, lbann.Trainer(mini_batch_size=8)


def test_grid_search_writes_one_file_per_point_and_runs(tmp_path, capsys):
    script = make_batch_script(work_dir=str(tmp_path), nodes=1, procs_per_node=2, scheduler="local")
    rows = grid_search(script, _experiment, procs_per_trainer=1, run=False,
                       learn_rate=[0.1, 0.01, 0.001], width=[6])
    # 3 points on 2 trainers: run 0 is full, run 1 repeats its only configuration
    assert [r[:2] for r in rows[1:]] == [[0, 0], [0, 1], [1, 0], [1, 1]]
    for name in ("run0.trainer0", "run0.trainer1", "run1.trainer0", "run1.trainer1"):
        assert os.path.exists(tmp_path / name)
    with open(tmp_path / "hyperparameters.csv") as f:
        table = list(csv.reader(f))
    assert table[0] == ["run_id", "trainer_id", "model_name", "learn_rate", "width"]
    assert [row[3] for row in table[1:]] == ["0.1", "0.01", "0.001", "0.001"]
    launches = [l for l in script.body if "--generate_multi_proto" in l]
    assert len(launches) == 2 and "run1.trainer0" in launches[1]
    # the driver picks the file of its own trainer
    from lbann_b200 import driver
    cwd = os.getcwd()
    os.chdir(tmp_path)
    try:
        rc = driver.main([f"--prototext={tmp_path}/run0.trainer0", "--generate_multi_proto",
                          "--procs_per_trainer=1", "--disable_cuda"])
    finally:
        os.chdir(cwd)
    assert rc == 0
    assert "training epoch 0 objective function" in capsys.readouterr().out


def test_profiling_regions_and_hierarchical_timers():
    import time
    import pytest
    from lbann_b200.utils import profiling as prof
    timers = prof.TimerMap("train")
    for _ in range(2):
        with timers.scope("epoch"):
            with timers.scope("forward"), prof.ProfRegion("forward"):
                time.sleep(0.002)
            with timers.scope("backward"):
                time.sleep(0.001)
    epoch = timers.children["epoch"]
    assert len(epoch.times) == 2 and set(epoch.children) == {"forward", "backward"}
    assert epoch.total() >= epoch.children["forward"].total() + epoch.children["backward"].total()
    text = timers.report()
    assert "epoch: total" in text and "    forward: total" in text
    prof.prof_region_begin("a")
    with pytest.raises(RuntimeError):
        prof.prof_region_end("b")
    info = prof.system_info()
    assert info["cpus"] >= 1 and "torch" in info


def test_saved_model_is_loaded_for_inference(tmp_path):
    """Train with the save-model callback, then rebuild the model through the embedding API
    with another mini-batch size and reproduce the trained model's outputs."""
    import numpy as np
    from lbann_b200 import inference
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.utils import options as opts
    o = opts.reset()
    o.set("disable_cuda", True)
    x = lbann.Input(data_field="samples")
    h = lbann.Relu(lbann.FullyConnected(x, num_neurons=7, has_bias=True, name="fc1"))
    y = lbann.FullyConnected(h, num_neurons=3, has_bias=True, name="fc2")
    probs = lbann.Softmax(y, name="probs")
    loss = lbann.CrossEntropy(probs, lbann.Input(data_field="labels"))
    model = lbann.Model(2, layers=list(lbann.traverse_layer_graph([x])),
                        objective_function=lbann.ObjectiveFunction([loss]),
                        callbacks=[lbann.CallbackSaveModel(dir=str(tmp_path / "saved"))])
    r = lbann.reader_pb2.Reader(name="synthetic", role="train", num_samples=16, synth_dimensions="5",
                                num_labels=3, fraction_of_data_to_use=1.0)
    dr = lbann.reader_pb2.DataReader()
    dr.reader.append(r)
    exp = lbann.proto.serialize.build_experiment(trainer=lbann.Trainer(mini_batch_size=8), model=model,
                                                 data_reader=dr, optimizer=lbann.SGD(learn_rate=0.1))
    os.makedirs(tmp_path / "saved", exist_ok=True)
    with open(tmp_path / "saved" / "experiment.prototext", "w") as f:
        from google.protobuf import text_format
        f.write(text_format.MessageToString(exp))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tr.train(m)
    data = np.random.RandomState(1).randn(6, 5).astype(np.float32)
    import torch
    with torch.no_grad():
        m.forward_prop({"samples": torch.from_numpy(data), "labels": torch.zeros(6, 3)}, "prediction")
        want = m.acts["probs"][0].numpy().copy()
    tr.shutdown()
    inference.initialize_lbann(["--disable_cuda"])
    h = inference.load_inference_model(str(tmp_path / "saved"), 4, {"samples": (5,), "labels": (3,)})
    got = h.infer(data, output_layer="probs")
    labels = h.infer(data, output_layer="probs", labels=True)
    inference.finalize_lbann(h)
    opts.reset()
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    assert labels.tolist() == want.argmax(1).tolist()


def test_cpu_binding_helpers(tmp_path, monkeypatch):
    """The core list of a GPU's NUMA node is parsed from sysfs; binding is skipped when the
    information is missing or disabled."""
    from lbann_b200.utils import affinity
    assert affinity.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert affinity.parse_cpulist("") == set()
    dev = tmp_path / "0000:1b:00.0"
    dev.mkdir()
    (dev / "local_cpulist").write_text("0-1,4\n")
    assert affinity.local_cpus_of("0000:1b:00.0", str(tmp_path)) == {0, 1, 4}
    assert affinity.local_cpus_of("0000:ff:00.0", str(tmp_path)) == set()
    monkeypatch.setattr(affinity, "gpu_pci_address", lambda i: "0000:1b:00.0")
    # fewer than four usable cores: nothing is changed
    assert affinity.bind_to_gpu(0, str(tmp_path)) is None
    monkeypatch.setenv("LBANN_DISABLE_NUMA_BIND", "1")
    assert affinity.bind_to_gpu(0, str(tmp_path)) is None


def test_operator_classes_through_lbann_ops():
    """``lbann.ops`` holds one class per operator message; an operator layer chains them."""
    import numpy as np
    import lbann_b200 as lbann
    assert {"Add", "Clamp", "Exp", "Scale", "Tanh"} <= set(lbann.ops.__all__)
    x = lbann.Input(data_field="samples")
    y = lbann.OperatorLayer(x, ops=[lbann.ops.Clamp(min=-1.0, max=0.5)], name="clamped")
    z = lbann.OperatorLayer(y, ops=[lbann.ops.Scale(constant=2.0)], name="scaled")
    data = np.linspace(-2, 2, 12, dtype=np.float32).reshape(3, 4)
    got = lbann.evaluate(z, data)
    np.testing.assert_allclose(got, 2.0 * np.clip(data, -1.0, 0.5), rtol=1e-6)
    import pytest
    with pytest.raises(ValueError, match="unknown argument"):
        lbann.ops.Clamp(minimum=0.0)
