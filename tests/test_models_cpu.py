"""Model zoo on CPU: every model builds through the front end, executes a few training
steps in the in-process executor and lowers the loss on a fixed synthetic batch."""
import math

import numpy as np
import pytest
import torch

import lbann_b200 as lbann
from lbann_b200.exec.trainer import ExecTrainer
from lbann_b200.utils import options as opts


def _reader(num, dims, distribution, label_classes=0, response_dims=None):
    r = lbann.reader_pb2.Reader()
    r.name = "synthetic"
    r.role = "train"
    r.shuffle = False
    r.fraction_of_data_to_use = 1.0
    r.synth_dimensions = " ".join(str(d) for d in dims)
    r.num_samples = num
    r.synth_distribution = distribution
    if label_classes:
        r.num_labels = label_classes
    if response_dims:
        r.synth_response_dimensions = " ".join(str(d) for d in response_dims)
    dr = lbann.reader_pb2.DataReader()
    dr.reader.append(r)
    return dr


def _train(model, reader, steps, mb, optimizer=None):
    o = opts.reset()
    o.set("disable_cuda", True)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=mb, random_seed=3), model=model, data_reader=reader,
        optimizer=optimizer or lbann.Adam(learn_rate=2e-3, beta1=0.9, beta2=0.99, eps=1e-8))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    losses = []
    for _ in range(steps):
        m.train_step(b.tensors, b.global_size)
        losses.append(float(m.last_objective))
    tr.shutdown()
    assert all(math.isfinite(v) for v in losses), losses
    return losses


def test_gpt_decoder_trains():
    from lbann_b200.models.transformer import construct_gpt_model
    torch.manual_seed(0)
    model = construct_gpt_model(vocab_size=48, seq_len=12, d_model=32, num_heads=4, num_layers=2,
                                ffn_dim=64)
    losses = _train(model, _reader(8, [13], "randint:48"), steps=20, mb=8)
    assert losses[0] == pytest.approx(math.log(48), rel=0.25)      # ~uniform prediction at start
    assert losses[-1] < 0.88 * losses[0], losses


def test_resnet18_trains_on_small_images():
    from lbann_b200.models import ResNet18, construct_classifier
    torch.manual_seed(0)
    model = construct_classifier(ResNet18(10, width=0.25), 10)
    losses = _train(model, _reader(8, [3, 32, 32], "normal", label_classes=10), steps=8, mb=8,
                    optimizer=lbann.SGD(learn_rate=0.05, momentum=0.9))
    assert losses[-1] < losses[0], losses


def test_resnet50_graph_has_the_published_size():
    """53 convolutions + 1 FC and 25.5 M parameters for 1000 classes."""
    from lbann_b200.models import ResNet50, construct_classifier
    model = construct_classifier(ResNet50(1000), 1000)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=2), model=model,
        data_reader=_reader(2, [3, 224, 224], "normal", label_classes=1000),
        optimizer=lbann.SGD(learn_rate=0.1, momentum=0.9))
    convs = [l for l in exp.model.layer if l.WhichOneof("layer_type") == "convolution"]
    assert len(convs) == 53
    o = opts.reset()
    o.set("disable_cuda", True)
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    n_params = sum(w.values.numel() for w in m.weights if "running" not in w.name)
    tr.shutdown()
    assert 25.4e6 < n_params < 25.7e6, n_params


def test_unet3d_trains():
    from lbann_b200.models import construct_unet3d_model
    torch.manual_seed(0)
    model = construct_unet3d_model(num_classes=3, base_channels=4, levels=2)
    r = _reader(2, [1, 8, 8, 8], "samples:normal responses:randint:3", response_dims=[8, 8, 8])
    losses = _train(model, r, steps=6, mb=2)
    assert losses[-1] < losses[0], losses


def test_recurrent_and_graph_modules_build_and_run():
    from lbann_b200 import modules
    torch.manual_seed(0)
    x = lbann.Input(data_field="samples")
    seq = lbann.Reshape(x, dims=[4, 6])
    sl = lbann.Slice(seq, axis=0, slice_points=[0, 1, 2, 3, 4])
    cell = modules.LSTMCell(5)
    h = lbann.Constant(value=0.0, num_neurons=[5])
    c = lbann.Constant(value=0.0, num_neurons=[5])
    for _ in range(4):
        step = lbann.Reshape(lbann.Identity(sl), dims=[6])
        h, (h, c) = cell(step, (h, c))
    adj = lbann.Constant(value=0.25, num_neurons=[4, 4])
    g = modules.DenseGCNConv(6, 3)(seq, adj)
    loss = lbann.Add(lbann.L2Norm2(h), lbann.L2Norm2(lbann.Reshape(g, dims=[12])))
    layers = list(lbann.traverse_layer_graph([x]))
    model = lbann.Model(1, layers=layers, objective_function=lbann.ObjectiveFunction([loss]))
    losses = _train(model, _reader(4, [24], "normal"), steps=5, mb=4,
                    optimizer=lbann.SGD(learn_rate=0.05))
    assert losses[-1] < losses[0], losses


def test_rotary_embedding_matches_the_rotation_formula():
    """q cos + rotate_half(q) sin per head, against the same written in numpy."""
    from lbann_b200.modules import RotaryPositionalEmbedding
    opts.reset().set("disable_cuda", True)
    S, H, P = 6, 2, 8
    rope = RotaryPositionalEmbedding(P, S, H)
    x = lbann.Reshape(lbann.Input(data_field="samples"), dims=[S, H * P])
    q, k, v = rope.apply_layer(x, x, x, S)
    data = np.random.RandomState(3).randn(3, S * H * P).astype(np.float32)
    out = lbann.evaluate([q, k], data, outputs=[q.name]).reshape(3, S, H, P)
    xs = data.reshape(3, S, H, P)
    inv = 1.0 / 10000.0 ** (np.arange(0, P, 2) / P)
    ang = np.outer(np.arange(S), inv)
    ang = np.concatenate([ang, ang], -1)[None, :, None, :]
    rot = np.concatenate([-xs[..., P // 2:], xs[..., :P // 2]], -1)
    want = xs * np.cos(ang) + rot * np.sin(ang)
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-5)
    assert v is x          # values are left alone unless embed_values is set


def test_gpt_with_rotary_positions_trains():
    from lbann_b200.models.transformer import construct_gpt_model
    torch.manual_seed(0)
    model = construct_gpt_model(vocab_size=48, seq_len=12, d_model=32, num_heads=4, num_layers=1,
                                ffn_dim=64, positional_encoding="rope")
    losses = _train(model, _reader(8, [13], "randint:48"), steps=20, mb=8)
    assert losses[-1] < 0.9 * losses[0], losses


def test_transformer_parallelism_switches_mark_the_graph():
    """--fsdp-mlp, --ffn-parallel, --lm-head-parallel and --layer-parallel act on the model
    by layer and weight names; the flags reach the serialised protobuf."""
    import argparse
    from lbann_b200.models import parallelism as par
    from lbann_b200.models.transformer import construct_gpt_model
    ap = argparse.ArgumentParser()
    par.add_transformer_parallelism_arguments(ap)

    model = construct_gpt_model(vocab_size=32, seq_len=8, d_model=16, num_heads=2, num_layers=4, ffn_dim=32)
    assert par.apply_fsdp_mlp(model, ap.parse_args(["--fsdp-mlp"])) == 8      # 4 blocks x (fc1, fc2)
    sharded = [w.name for l in model.layers for w in l.weights if w.sharded]
    assert sharded and all(n.endswith(("_fc1_matrix", "_fc2_matrix")) for n in sharded)
    with pytest.raises(ValueError):
        par.apply_fsdp_mlp(model, ap.parse_args(["--fsdp-mlp", "--ffn-parallel"]))

    model = construct_gpt_model(vocab_size=32, seq_len=8, d_model=16, num_heads=2, num_layers=4, ffn_dim=32)
    changed = par.apply_ffn_model_parallelism(model, ap.parse_args(["--ffn-parallel"]), blocks=[1, 3])
    assert len(changed) == 4 and all("_block1_" in n or "_block3_" in n for n in changed)
    head = next(l for l in model.layers if l.name.startswith("gpt_head"))
    tail = par.apply_lm_head_model_parallelism(model, head, ap.parse_args(["--lm-head-parallel"]))
    assert head.name in tail and "loss" in tail and "gpt_embed" not in tail
    grids = par.apply_layer_parallelism(model, ap.parse_args(["--layer-parallel", "--lp-count", "2"]))
    assert grids == 2
    tags = {l.name: (l.grid_tag or {}).get("value", 0) for l in model.layers}
    assert tags[next(n for n in tags if "_block0_" in n)] == 1
    assert tags[next(n for n in tags if "_block3_" in n)] == 2
    msg = model.export_proto()
    layouts = {l.name: l.data_layout for l in msg.layer}
    assert layouts[head.name] == "model_parallel"
    assert any(l.grid_tag.value == 2 for l in msg.layer)
