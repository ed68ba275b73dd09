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
