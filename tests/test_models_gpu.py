"""Model zoo on a GPU in 16-bit precision: the native kernels (tcgen05 GEMM / convolution,
layer norm, softmax, fused softmax-cross-entropy, batch norm, fused optimizer) carry a few
training steps of every model family."""
import math

import pytest
import torch

import lbann_b200 as lbann
from lbann_b200.exec.trainer import ExecTrainer
from lbann_b200.ops import native
from lbann_b200.utils import options as opts
from test_models_cpu import _reader

pytestmark = pytest.mark.gpu


def _train_gpu(model, reader, steps, mb, dtype, optimizer=None, graph=False):
    o = opts.reset()
    o.set("default_dtype", dtype)
    if graph:
        o.set("use_cuda_graph", True)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=mb, random_seed=3), model=model, data_reader=reader,
        optimizer=optimizer or lbann.Adam(learn_rate=2e-3, beta1=0.9, beta2=0.99, eps=1e-8))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    n0 = native.launches()
    losses = []
    for _ in range(steps):
        m.train_step(b.tensors, b.global_size)
        losses.append(float(m.last_objective))
    assert native.consume_status() == 0
    assert native.launches() > n0, "no native kernel ran"
    if graph:
        assert m._graph_mode and any("graph" in e for e in m._graphs.values()), "step was not captured"
    tr.shutdown()
    assert all(math.isfinite(v) for v in losses), losses
    return losses


def test_gpt_bf16():
    from lbann_b200.models.transformer import construct_gpt_model
    torch.manual_seed(0)
    model = construct_gpt_model(vocab_size=256, seq_len=64, d_model=128, num_heads=4, num_layers=2,
                                ffn_dim=512)
    losses = _train_gpu(model, _reader(8, [65], "randint:256"), steps=20, mb=8, dtype="bf16")
    assert losses[0] == pytest.approx(math.log(256), rel=0.25)
    assert losses[-1] < 0.9 * losses[0], losses


def test_resnet18_bf16():
    from lbann_b200.models import ResNet18, construct_classifier
    torch.manual_seed(0)
    model = construct_classifier(ResNet18(16, width=0.5), 16)
    losses = _train_gpu(model, _reader(16, [3, 64, 64], "normal", label_classes=16), steps=10, mb=16,
                        dtype="bf16", optimizer=lbann.SGD(learn_rate=0.05, momentum=0.9))
    assert losses[-1] < losses[0], losses


def test_unet3d_fp16():
    from lbann_b200.models import construct_unet3d_model
    torch.manual_seed(0)
    model = construct_unet3d_model(num_classes=3, base_channels=8, levels=2)
    r = _reader(2, [1, 32, 32, 32], "samples:normal responses:randint:3", response_dims=[32, 32, 32])
    losses = _train_gpu(model, r, steps=8, mb=2, dtype="fp16")
    assert losses[-1] < losses[0], losses


def test_attention_score_fusion_matches_unfused(monkeypatch):
    """Folding 1/sqrt(d) and the causal mask into the softmax kernel does not change the
    training trajectory beyond 16-bit rounding."""
    from lbann_b200.models.transformer import construct_gpt_model

    def run():
        torch.manual_seed(0)
        model = construct_gpt_model(vocab_size=128, seq_len=32, d_model=64, num_heads=4, num_layers=2,
                                    ffn_dim=128, name="gptf")
        return _train_gpu(model, _reader(8, [33], "randint:128"), steps=6, mb=8, dtype="bf16")

    fused = run()
    monkeypatch.setenv("LBANN_DISABLE_ATTENTION_FUSION", "1")
    plain = run()
    for a, b in zip(fused, plain):
        assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (fused, plain)



@pytest.mark.parametrize("family", ["cosmoflow_amp", "gpt"])
def test_cuda_graph_replay_matches_eager_steps(family):
    """The training step captured as a CUDA graph (after three ordinary steps) and replayed
    gives the losses of the step-by-step run: same kernels, same order, device-side
    optimizer step counter and loss-scale schedule."""
    def build():
        torch.manual_seed(0)
        if family == "gpt":
            from lbann_b200.models.transformer import construct_gpt_model
            m = construct_gpt_model(vocab_size=256, seq_len=64, d_model=128, num_heads=4, num_layers=2,
                                    ffn_dim=512)
            return m, _reader(8, [65], "randint:256"), "bf16"
        from lbann_b200.models.cosmoflow import construct_cosmoflow_model, synthetic_reader
        m = construct_cosmoflow_model(32, 4, 4, num_epochs=1, channels=(16, 32, 32), pool_mode="max",
                                      conv_bias=False, fc_sizes=(64, 32))
        m.amp = lbann.AmpOptions(enabled=True, init_scale=1024.0)
        return m, synthetic_reader(8, 32, 4, 4), "fp16"

    model, reader, dt = build()
    sgd = lambda: lbann.Adam(learn_rate=1e-4, beta1=0.9, beta2=0.99, eps=1e-8)      # noqa: E731
    eager = _train_gpu(model, reader, steps=10, mb=8, dtype=dt, optimizer=sgd())
    model, reader, dt = build()
    again = _train_gpu(model, reader, steps=10, mb=8, dtype=dt, optimizer=sgd())
    model, reader, dt = build()
    replay = _train_gpu(model, reader, steps=10, mb=8, dtype=dt, optimizer=sgd(), graph=True)
    # tolerance: what two step-by-step runs differ by (fp32 atomics in the filter gradients)
    noise = max(abs(a - b) for a, b in zip(eager, again))
    for a, b in zip(eager, replay):
        assert abs(a - b) <= max(5.0 * noise, 2e-3 * max(1.0, abs(a))), (eager, again, replay)


def test_learning_rate_change_reaches_a_captured_step():
    """A learning-rate schedule keeps working under graph replay: the optimizer kernel reads
    its hyper-parameters from a device table that is refreshed before a replay."""
    from lbann_b200.models.transformer import construct_gpt_model
    torch.manual_seed(0)
    o = opts.reset()
    o.set("default_dtype", "bf16")
    o.set("use_cuda_graph", True)
    model = construct_gpt_model(vocab_size=128, seq_len=32, d_model=64, num_heads=2, num_layers=1, ffn_dim=128)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=4, random_seed=3), model=model,
        data_reader=_reader(4, [33], "randint:128"), optimizer=lbann.SGD(learn_rate=0.05))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    for _ in range(6):
        m.train_step(b.tensors, b.global_size)
    assert any("graph" in e for e in m._graphs.values())
    before = m.arena.master.detach().clone()
    m.train_step(b.tensors, b.global_size)
    moved = float((m.arena.master - before).abs().max())
    for s in m.arena.slots:
        s.hp["learn_rate"] = 0.0
    before = m.arena.master.detach().clone()
    m.train_step(b.tensors, b.global_size)
    frozen = float((m.arena.master - before).abs().max())
    tr.shutdown()
    assert native.consume_status() == 0
    assert moved > 0.0 and frozen == 0.0, (moved, frozen)


def test_kfac_on_gpu_beats_plain_sgd():
    """K-FAC preconditioning (Kronecker factors, damped inverses) with the layers' native
    kernels underneath reaches a lower objective than plain SGD in the same epochs."""
    from test_algorithms_cpu import _fit
    sgd = lbann.BatchedIterativeOptimizer("sgd", epoch_count=3)
    kfac = lbann.KFAC("kfac", sgd, damping_act="1e-2", damping_err="1e-2", kronecker_decay=0.9,
                      update_intervals="1", compute_interval=1)
    plain = _fit(sgd, cuda=True)
    second = _fit(kfac, cuda=True)
    assert native.consume_status() == 0
    assert math.isfinite(second) and second < plain, (plain, second)
