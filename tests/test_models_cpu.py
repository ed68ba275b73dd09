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


def _graph_forward(build, n_nodes, feat, n_edges, extra=0, seed=0):
    """Builds a model whose input sample is [node features | source | target | extra],
    runs one forward pass and returns (model, input tensors, activation getter)."""
    o = opts.reset()
    o.set("disable_cuda", True)
    width = n_nodes * feat + 2 * n_edges + extra
    x = lbann.Input(data_field="samples")
    parts = lbann.Slice(x, axis=0, slice_points=[0, n_nodes * feat, n_nodes * feat + n_edges,
                                                 n_nodes * feat + 2 * n_edges] + ([width] if extra else []))
    nodes = lbann.Reshape(lbann.Identity(parts), dims=[n_nodes, feat])
    src = lbann.Identity(parts)
    dst = lbann.Identity(parts)
    rest = lbann.Identity(parts) if extra else None
    out = build(nodes, src, dst, rest)
    out = lbann.Identity(out, name="graph_out")
    loss = lbann.L2Norm2(lbann.Reshape(out, dims=[-1]))
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=2, random_seed=seed + 1), model=model,
        data_reader=_reader(2, [width], "normal"), optimizer=lbann.SGD(learn_rate=0.01))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    g = torch.Generator().manual_seed(seed)
    feats = torch.randn(2, n_nodes, feat, generator=g)
    s = torch.randint(0, n_nodes, (2, n_edges), generator=g).float()
    t = torch.randint(0, n_nodes, (2, n_edges), generator=g).float()
    s[:, -1] = -1                   # a padding edge
    t[:, -1] = -1
    ex = torch.randn(2, extra, generator=g) if extra else torch.zeros(2, 0)
    sample = torch.cat([feats.reshape(2, -1), s, t, ex], 1)
    m.forward_prop({"samples": sample}, "validation")
    return tr, m, feats, s.long(), t.long(), ex


def _propagate(msg, s, t, n_nodes):
    """out[b, s[e]] += msg[b, t[e]] for edges with valid indices."""
    out = torch.zeros(msg.shape[0], n_nodes, msg.shape[2])
    for b in range(msg.shape[0]):
        for e in range(s.shape[1]):
            if s[b, e] >= 0 and t[b, e] >= 0:
                out[b, s[b, e]] += msg[b, t[b, e]]
    return out


def test_sparse_graph_convolutions_match_their_formulas():
    from lbann_b200 import modules
    N, F, E, C = 5, 4, 9, 3
    # GCN: sum over neighbours of relu(W x_j + b)
    tr, m, x, s, t, _ = _graph_forward(
        lambda nodes, src, dst, _: modules.GCNConv(F, C, N, name="gcn")(nodes, src, dst), N, F, E)
    W = m.weights_by_name["gcn_weights"].values.detach().reshape(C, F)
    b = m.weights_by_name["gcn_bias_weights"].values.detach().reshape(C)
    ref = _propagate(torch.relu(x @ W.t() + b), s, t, N)
    torch.testing.assert_close(m.activation("graph_out").float(), ref, rtol=1e-5, atol=1e-5)
    tr.shutdown()
    # GraphConv: relu(W1 x_i) + sum relu(W2 x_j + b)
    tr, m, x, s, t, _ = _graph_forward(
        lambda nodes, src, dst, _: modules.GraphConv(F, C, N, name="gc")(nodes, src, dst), N, F, E, seed=1)
    wn = {w.name: w.values.detach() for w in m.weights}
    W1 = wn["gc_ID_FC_layer_matrix"].reshape(C, F)
    W2 = wn["gc_Message_FC_layer_matrix"].reshape(C, F)
    b2 = wn["gc_Message_FC_layer_bias"].reshape(C)
    ref = torch.relu(x @ W1.t()) + _propagate(torch.relu(x @ W2.t() + b2), s, t, N)
    torch.testing.assert_close(m.activation("graph_out").float(), ref, rtol=1e-5, atol=1e-5)
    tr.shutdown()
    # GIN on an edge list with a one-layer network
    tr, m, x, s, t, _ = _graph_forward(
        lambda nodes, src, dst, _: modules.SparseGINConv(
            [modules.ChannelwiseFullyConnectedModule(C, bias=False, name="gin_fc")], F, C, N, eps=0.5,
            name="gin")(nodes, src, dst), N, F, E, seed=2)
    Wg = m.weights_by_name["gin_fc_matrix"].values.detach().reshape(C, F)
    ref = (1.5 * x + _propagate(x, s, t, N)) @ Wg.t()
    torch.testing.assert_close(m.activation("graph_out").float(), ref, rtol=1e-5, atol=1e-5)
    tr.shutdown()
    opts.reset()


def test_gated_graph_and_edge_conditioned_convolutions():
    from lbann_b200 import modules
    N, F, E, C, EF = 4, 3, 6, 5, 2
    # GatedGraphConv: padded input, one round: h' = GRU(sum_j W h_j, h)
    tr, m, x, s, t, _ = _graph_forward(
        lambda nodes, src, dst, _: modules.GatedGraphConv(F, C, N, num_layers=1, name="ggc")(nodes, src, dst),
        N, F, E, seed=3)
    wn = {w.name: w.values.detach() for w in m.weights}
    h = torch.cat([x, torch.zeros(2, N, C - F)], 2)
    Wm = wn["ggc_message_0_matrix"].reshape(C, C)
    msg = _propagate(h @ Wm.t(), s, t, N)
    Wih, bih = wn["ggc_gru_ih_fc_matrix"].reshape(3 * C, C), wn["ggc_gru_ih_fc_bias"].reshape(3 * C)
    Whh, bhh = wn["ggc_gru_hh_fc_matrix"].reshape(3 * C, C), wn["ggc_gru_hh_fc_bias"].reshape(3 * C)
    gi, gh = msg @ Wih.t() + bih, h @ Whh.t() + bhh
    r = torch.sigmoid(gi[..., :C] + gh[..., :C])
    z = torch.sigmoid(gi[..., C:2 * C] + gh[..., C:2 * C])
    n = torch.tanh(gi[..., 2 * C:] + r * gh[..., 2 * C:])
    ref = (1 - z) * n + z * h
    torch.testing.assert_close(m.activation("graph_out").float(), ref, rtol=1e-5, atol=1e-5)
    tr.shutdown()

    # NNConv: relu(Theta x_i) + sum_{e: s[e] = i} x_{t[e]} . reshape(W_e edge_feat[e])
    def build(nodes, src, dst, rest):
        edge_feats = lbann.Reshape(rest, dims=[E, EF])
        nbr = lbann.Reshape(modules.GraphExpand(nodes, dst), dims=[E, 1, F])
        nn = [modules.ChannelwiseFullyConnectedModule(F * C, bias=False, name="edge_fc")]
        return modules.NNConv(nn, N, E, F, C, EF, name="nnc")(nodes, nbr, edge_feats, src)
    tr, m, x, s, t, ex = _graph_forward(build, N, F, E, extra=E * EF, seed=4)
    wn = {w.name: w.values.detach() for w in m.weights}
    We = wn["edge_fc_matrix"].reshape(F * C, EF)
    Wn = wn["nnc_node_weights_matrix"].reshape(C, F)
    ef = ex.reshape(2, E, EF)
    ref = torch.relu(x @ Wn.t())
    for b in range(2):
        for e in range(E):
            if s[b, e] >= 0 and t[b, e] >= 0:
                theta = (We @ ef[b, e]).reshape(F, C)
                ref[b, s[b, e]] += x[b, t[b, e]] @ theta
    torch.testing.assert_close(m.activation("graph_out").float(), ref, rtol=1e-5, atol=1e-5)
    tr.shutdown()
    opts.reset()


def test_roberta_matches_the_transformers_implementation(tmp_path):
    """A small RoBERTa with its parameters exported to ``.npy``: last hidden states and the
    pooled output equal those of ``transformers.RobertaModel`` on ids with padding."""
    transformers = pytest.importorskip("transformers")
    from lbann_b200.models.roberta import RoBERTa, RobertaConfig
    torch.manual_seed(0)
    S = 10
    kw = dict(vocab_size=40, hidden_size=16, num_hidden_layers=2, num_attention_heads=4, intermediate_size=32,
              max_position_embeddings=S + 2, type_vocab_size=1, pad_token_id=1, layer_norm_eps=1e-5,
              hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    hf = transformers.RobertaModel(transformers.RobertaConfig(**kw)).eval()
    for name, p in hf.state_dict().items():
        if p.dtype.is_floating_point:
            np.save(tmp_path / f"{name}.npy", p.detach().numpy())
    o = opts.reset()
    o.set("disable_cuda", True)
    ids_in = lbann.Input(data_field="samples")
    sl = lbann.Slice(ids_in, axis=0, slice_points=[0, S, 2 * S])
    ids, amask = lbann.Identity(sl), lbann.Identity(sl)
    hidden, pooled = RoBERTa(RobertaConfig(**kw), S, load_weights=str(tmp_path))(ids, attention_mask=amask)
    hidden = lbann.Identity(hidden, name="hidden_out")
    pooled = lbann.Identity(pooled, name="pooled_out")
    loss = lbann.Add(lbann.L2Norm2(lbann.Reshape(hidden, dims=[-1])), lbann.L2Norm2(pooled))
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([ids_in])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=3), model=model, data_reader=_reader(3, [2 * S], "normal"),
        optimizer=lbann.SGD(learn_rate=0.0))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tok = torch.randint(2, 40, (3, S))
    tok[0, 7:] = 1                      # padding at the end of the first sequence
    tok[2, 4:] = 1
    att = (tok != 1).long()
    m.forward_prop({"samples": torch.cat([tok, att], 1).float()}, "validation")
    with torch.no_grad():
        ref = hf(input_ids=tok, attention_mask=att)
    got_h, got_p = m.activation("hidden_out").float(), m.activation("pooled_out").float()
    keep = att.bool()
    torch.testing.assert_close(got_h[keep], ref.last_hidden_state[keep], rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(got_p, ref.pooler_output, rtol=2e-4, atol=2e-4)
    tr.shutdown()
    opts.reset()


# ------------------------------------------------------------------ application models
def test_autoencoders_reduce_the_reconstruction_error():
    from lbann_b200.models.applications import construct_autoencoder
    torch.manual_seed(0)
    dense = construct_autoencoder((1, 12, 12), "dense", hidden=(64, 32, 8))
    losses = _train(dense, _reader(8, [1, 12, 12], "uniform"), steps=25, mb=8)
    assert losses[-1] < 0.9 * losses[0], losses
    conv = construct_autoencoder((1, 12, 12), "conv")
    losses = _train(conv, _reader(8, [1, 12, 12], "uniform"), steps=25, mb=8)
    assert losses[-1] < 0.95 * losses[0], losses


def test_vae_objective_is_reconstruction_plus_kl():
    from lbann_b200.models.applications import construct_vae
    torch.manual_seed(0)
    model = construct_vae(input_size=36, hidden=(32, 16), latent=4)
    losses = _train(model, _reader(8, [36], "uniform"), steps=30, mb=8)
    assert losses[0] > 0.8 * 36 * math.log(2)       # at least ~log 2 per pixel at the start, plus the KL term
    assert losses[-1] < 0.9 * losses[0], losses


def test_gan_alternates_discriminator_and_generator_updates():
    from lbann_b200.models.applications import construct_gan
    torch.manual_seed(0)
    model = construct_gan(sample_size=36, noise_size=4, hidden=(16, 16))
    o = opts.reset()
    o.set("disable_cuda", True)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=3), model=model,
        data_reader=_reader(8, [36], "uniform"), optimizer=lbann.Adam(learn_rate=1e-3, beta1=0.5, beta2=0.99, eps=1e-8))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")

    def snap(prefix):
        return {w.name: w.values.detach().clone() for w in m.weights if w.name.startswith(prefix)}
    moved = []
    for step in range(4):
        g0, d0 = snap("gen_"), snap("disc_")
        for cb in m.callbacks:
            cb.on_batch_begin(m)
        m.train_step(b.tensors, b.global_size)
        m.ctx.step += 1
        g1, d1 = snap("gen_"), snap("disc_")
        moved.append((any(not torch.equal(g0[k], g1[k]) for k in g0), any(not torch.equal(d0[k], d1[k]) for k in d0)))
    tr.shutdown()
    # step 0: discriminator only; step 1: generator only; and so on
    assert moved == [(False, True), (True, False), (False, True), (True, False)], moved


def test_densenet_small_builds_and_trains():
    from lbann_b200.models.applications import construct_densenet
    torch.manual_seed(0)
    model = construct_densenet(num_classes=5, growth=4, blocks=(2, 2), init_features=8, small_input=True)
    losses = _train(model, _reader(8, [3, 8, 8], "normal", label_classes=5), steps=15, mb=8)
    assert losses[-1] < losses[0], losses
    full = construct_densenet()            # DenseNet-121: 58 dense layers x 2 convs + stem + 3 transitions
    convs = [l for l in lbann.traverse_layer_graph(full.layers) if type(l).__name__ == "Convolution"]
    assert len(convs) == 2 * (6 + 12 + 24 + 16) + 1 + 3


def test_char_rnn_learns_a_repeating_sequence():
    from lbann_b200.models.applications import construct_char_rnn
    torch.manual_seed(0)
    model = construct_char_rnn(vocab_size=11, sequence_length=9, embedding_size=8, hidden_size=16)
    losses = _train(model, _reader(4, [9], "randint:11"), steps=40, mb=4,
                    optimizer=lbann.Adam(learn_rate=2e-2, beta1=0.9, beta2=0.99, eps=1e-8))
    assert losses[0] == pytest.approx(math.log(11), rel=0.3)
    assert losses[-1] < 0.7 * losses[0], losses


def test_dense_gcn_siamese_candle_and_jag_models_train():
    from lbann_b200.models.applications import (construct_candle_combo, construct_dense_gcn,
                                                construct_jag_wae, construct_siamese)
    torch.manual_seed(0)
    gcn = construct_dense_gcn(num_nodes=6, num_features=3, num_classes=2, hidden=(8, 8))
    losses = _train(gcn, _reader(8, [6 * 3 + 36], "uniform", label_classes=2), steps=20, mb=8)
    assert losses[-1] < losses[0], losses
    siam = construct_siamese(num_patches=3, patch_dims=(1, 8, 8), num_classes=6, embed=8)
    losses = _train(siam, _reader(8, [3, 8, 8], "normal", label_classes=6), steps=20, mb=8)
    assert losses[-1] < losses[0], losses
    combo = construct_candle_combo(cell_features=5, drug_features=7, hidden=(16, 16))
    losses = _train(combo, _reader(8, [19], "normal", response_dims=[1]), steps=20, mb=8)
    assert losses[-1] < losses[0], losses
    wae = construct_jag_wae(sample_size=24, latent=3, enc_hidden=(16, 8), disc_hidden=(8,))
    losses = _train(wae, _reader(8, [24], "normal"), steps=20, mb=8)
    assert losses[-1] < losses[0], losses


def test_node2vec_voxel_autoencoder_and_image_regressor_train(tmp_path):
    from lbann_b200.models.applications import (construct_image_regressor, construct_node2vec,
                                                construct_voxel_autoencoder)
    torch.manual_seed(0)
    # a ring graph: walks visit neighbours, so neighbours' embeddings align
    n = 12
    (tmp_path / "ring.txt").write_text("".join(f"{i} {(i + 1) % n}\n" for i in range(n)))
    r = lbann.reader_pb2.Reader()
    r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "node2vec", "train", False, 1.0
    r.node2vec.graph_file, r.node2vec.epoch_size, r.node2vec.walk_length = str(tmp_path / "ring.txt"), 16, 5
    r.node2vec.return_param = r.node2vec.inout_param = 1.0
    r.node2vec.num_negative_samples = 3
    dr = lbann.reader_pb2.DataReader()
    dr.reader.append(r)
    model = construct_node2vec(num_vertices=n, walk_length=5, num_negative_samples=3, latent_dim=8)
    losses = _train(model, dr, steps=40, mb=8, optimizer=lbann.SGD(learn_rate=0.5))
    assert losses[-1] < 0.9 * losses[0], losses
    ae = construct_voxel_autoencoder(channels=2, size=8, base=4, latent=8)
    losses = _train(ae, _reader(8, [2, 8, 8, 8], "uniform"), steps=20, mb=8)
    assert losses[-1] < losses[0], losses
    reg = construct_image_regressor(input_dims=(1, 32, 32), num_outputs=3)
    losses = _train(reg, _reader(8, [1, 32, 32], "normal", response_dims=[3]), steps=15, mb=8)
    assert losses[-1] < losses[0], losses
