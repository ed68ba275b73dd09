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
