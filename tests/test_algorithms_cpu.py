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


def test_model_surgery_keeps_weights_and_changes_the_graph():
    """insert / replace / remove / swap on a set-up model: the graph changes, weights whose
    name and shape survive keep values and optimizer state, and training carries on."""
    import torch
    import lbann_b200 as lbann
    from lbann_b200.exec import surgery
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.proto import lbann_pb2 as pb
    from lbann_b200.utils import options as opts
    from test_models_cpu import _reader
    o = opts.reset()
    o.set("disable_cuda", True)
    x = lbann.Input(data_field="samples")
    h = lbann.FullyConnected(x, num_neurons=6, name="fc1", weights=[lbann.Weights(name="w1"), lbann.Weights(name="b1")],
                             has_bias=True)
    a = lbann.Relu(h, name="act1")
    y = lbann.FullyConnected(a, num_neurons=3, name="fc2", weights=[lbann.Weights(name="w2")])
    loss = lbann.MeanSquaredError(y, lbann.Input(data_field="responses"), name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=4), model=model,
        data_reader=_reader(8, [5], "normal", response_dims=[3]), optimizer=lbann.Adam(learn_rate=0.01))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    for _ in range(3):
        m.train_step(b.tensors, b.global_size)
    w1 = m.weights_by_name["w1"].values.detach().clone()
    mom = {k: v.clone() for k, v in m.weights_by_name["w1"].optimizer_state().items()}

    # replace the activation
    new = pb.Layer(name="act1")
    new.leaky_relu.negative_slope = 0.2
    m2 = surgery.replace_layer(tr, m, "act1", new)
    assert m2.layer("act1").type == "leaky_relu" and m2 in tr.models and m not in tr.models
    assert torch.equal(m2.weights_by_name["w1"].values, w1)
    for k, v in m2.weights_by_name["w1"].optimizer_state().items():
        assert torch.equal(v, mom[k]), k
    # insert a layer behind it, then take it out again
    ins = pb.Layer(name="drop_in")
    ins.identity.SetInParent()
    m3 = surgery.insert_layer(tr, m2, ins, after="act1")
    assert [p.name for p in m3.layer("fc2").parents] == ["drop_in"]
    assert [p.name for p in m3.layer("drop_in").parents] == ["act1"]
    m4 = surgery.remove_layer(tr, m3, "drop_in")
    assert [p.name for p in m4.layer("fc2").parents] == ["act1"]
    assert "drop_in" not in m4.layers_by_name
    assert torch.equal(m4.weights_by_name["w2"].values, m2.weights_by_name["w2"].values)
    before = float(m4.train_step(b.tensors, b.global_size))
    for _ in range(5):
        after = float(m4.train_step(b.tensors, b.global_size))
    assert after < before
    # swap two neighbouring activations: fc1 -> act1 -> act2 -> fc2 becomes fc1 -> act2 -> act1 -> fc2
    t = pb.Layer(name="act2")
    t.elu.alpha = 1.0
    m5 = surgery.insert_layer(tr, m4, t, after="act1")
    m6 = surgery.swap_layers(tr, m5, "act1", "act2")
    assert [p.name for p in m6.layer("act2").parents] == ["fc1"]
    assert [p.name for p in m6.layer("act1").parents] == ["act2"]
    assert [p.name for p in m6.layer("fc2").parents] == ["act1"]
    assert len(tr.models) == 1
    float(m6.train_step(b.tensors, b.global_size))
    tr.shutdown()
    opts.reset()


def _bn_mlp():
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    h = lbann.FullyConnected(x, num_neurons=12, has_bias=True, name="fc1")
    h = lbann.BatchNormalization(h, name="bn1", epsilon=1e-5)
    y = lbann.FullyConnected(lbann.Tanh(h), num_neurons=3, has_bias=True, name="fc2")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    return lbann.Model(2, layers=list(lbann.traverse_layer_graph([x, t])),
                       objective_function=lbann.ObjectiveFunction([loss]))


def test_kfac_batch_norm_block_and_eigen_inverses():
    """The batch-norm block: per-sample (scale, bias) gradients add up to the layer's
    gradients, the preconditioned gradient is F^-1 g with the damped Fisher matrix of those
    samples, and training with eigen-decomposed inverses stays finite and improves."""
    from lbann_b200.exec.kfac import KFAC
    o = opts.reset()
    o.set("disable_cuda", True)
    sgd = lbann.BatchedIterativeOptimizer("sgd", epoch_count=2)
    algo = lbann.KFAC("kfac", sgd, damping_act="1e-2", damping_err="1e-2", damping_bn_err="3e-2",
                      kronecker_decay=0.9, update_intervals="1", compute_interval=1, use_eigen_decomposition=True)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=16, random_seed=9, training_algo=algo), model=_bn_mlp(),
        data_reader=_reader(64, [8], "normal", response_dims=[3]),
        optimizer=lbann.SGD(learn_rate=0.05, momentum=0.0))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    k = tr.algorithm
    assert isinstance(k, KFAC) and k.use_eigen
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    # one step by hand up to the preconditioner
    k._setup(m)
    k._ready = True
    assert set(k.blocks) == {"fc1", "bn1", "fc2"}
    m.clear_gradients()
    m.forward_prop(b.tensors, "training", b.global_size, 0)
    k._capture(m)
    obj = m.local_objective()
    m.backward_prop(obj)
    bn = m.layer("bn1")
    raw = torch.cat([bn.scale.handle.grad.reshape(-1), bn.bias.handle.grad.reshape(-1)]).clone()
    gs = k.blocks["bn1"].bn_sample_gradients(b.global_size)
    torch.testing.assert_close(gs.sum(0) / b.global_size, raw, rtol=1e-4, atol=1e-6)
    k._precondition(m, 0, b.global_size)
    Fm = gs.t() @ gs / gs.shape[0]
    expect = torch.linalg.solve(Fm + 3e-2 * torch.eye(Fm.shape[0]), raw)
    got = torch.cat([bn.scale.handle.grad.reshape(-1), bn.bias.handle.grad.reshape(-1)])
    torch.testing.assert_close(got, expect, rtol=1e-3, atol=1e-5)
    tr.shutdown()
    # and the whole loop
    first = _fit_model(_bn_mlp, sgd)
    second = _fit_model(_bn_mlp, algo)
    assert math.isfinite(second) and second < first, (first, second)


def _fit_model(make, algo, epochs=2):
    o = opts.reset()
    o.set("disable_cuda", True)
    torch.manual_seed(0)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=16, random_seed=9, training_algo=algo), model=make(),
        data_reader=_reader(64, [8], "normal", response_dims=[3]),
        optimizer=lbann.SGD(learn_rate=0.05, momentum=0.0))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tr.train(m, num_epochs=epochs)
    obj, _, _ = m.reduce_statistics("training")
    tr.shutdown()
    return obj


def test_torch_lowering_of_functions_parameters_and_token_models():
    """fx lowering beyond Sequential stacks: residual adds, concatenation, a parameter used
    directly in forward(), mean / transpose / matmul / softmax over sample dimensions, and an
    embedding + transposed convolution model; outputs equal PyTorch's."""
    import torch.nn as nn
    import torch.nn.functional as F
    import lbann_b200.torch as lt
    opts.reset().set("disable_cuda", True)
    torch.manual_seed(0)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.q, self.k, self.v = nn.Linear(8, 8), nn.Linear(8, 8), nn.Linear(8, 8)
            self.gate = nn.Parameter(torch.randn(5, 8) * 0.1)
            self.norm = nn.LayerNorm(8)
            self.head = nn.Linear(16, 3)

        def forward(self, input):                      # [N, 5, 8]
            q, k, v = self.q(input), self.k(input), self.v(input)
            att = torch.softmax(torch.matmul(q, k.transpose(1, 2)) / 8 ** 0.5, dim=-1)
            h = self.norm(input + torch.matmul(att, v) * self.gate)
            pooled = torch.cat([h.mean(dim=1), F.silu(h).mean(dim=1)], dim=1)
            return self.head(pooled)

    net = Block()
    x = torch.randn(4, 5, 8)
    got = lbann.evaluate(lt.compile(net, input=x)[0], x.numpy())
    torch.testing.assert_close(torch.from_numpy(got).reshape(4, 3), net(x).detach(), rtol=1e-4, atol=1e-5)

    class Tokens(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(11, 6)
            self.up = nn.ConvTranspose1d(6, 4, 2, stride=2)
            self.pool = nn.AdaptiveAvgPool2d(1)

        def forward(self, input):                      # [N, 7] token ids
            h = self.emb(input).permute(0, 2, 1)       # [N, 6, 7]
            return torch.exp(-self.up(h)).reshape(-1, 4, 14)

    net = Tokens()
    ids = torch.randint(0, 11, (3, 7))
    got = lbann.evaluate(lt.compile(net, input=ids)[0], ids.float().numpy())
    torch.testing.assert_close(torch.from_numpy(got).reshape(3, 4, 14), net(ids).detach(), rtol=1e-4, atol=1e-5)


def test_kfac_gru_block_preconditions_every_gate():
    """The GRU block: factors from the captured inputs / previous hidden states and the
    per-gate error signals; the preconditioned gradient of gate k is G_k^-1 [dW_k | db_k] A^-1
    with the damped factors, and a K-FAC run on a GRU regression stays finite and improves."""
    from lbann_b200.exec.kfac import KFAC
    from lbann_b200.modules.rnn import GRU
    o = opts.reset()
    o.set("disable_cuda", True)
    T, I, H = 5, 3, 4

    def model():
        x = lbann.Reshape(lbann.Input(data_field="samples"), dims=[T, I])
        h0 = lbann.Constant(value=0.0, num_neurons=[1, H])
        y = GRU(H, name="g")(x, h0)
        pred = lbann.FullyConnected(lbann.Reshape(y, dims=[T * H]), num_neurons=2, has_bias=True, name="head")
        loss = lbann.MeanSquaredError(pred, lbann.Input(data_field="responses"))
        return lbann.Model(2, layers=list(lbann.traverse_layer_graph(x)), objective_function=lbann.ObjectiveFunction([loss]))

    sgd = lbann.BatchedIterativeOptimizer("sgd", epoch_count=2)
    algo = lbann.KFAC("kfac", sgd, damping_act="1e-2", damping_err="1e-2", kronecker_decay=0.9,
                      update_intervals="1", compute_interval=1)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=11, training_algo=algo), model=model(),
        data_reader=_reader(32, [T * I], "normal", response_dims=[2]), optimizer=lbann.SGD(learn_rate=0.05))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    k = tr.algorithm
    assert isinstance(k, KFAC)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    b = dc.next_batch("training")
    k._setup(m)
    k._ready = True
    gru = next(l for l in m.layers if l.type == "gru")
    assert gru.name in k.blocks and gru.kfac_capture
    m.clear_gradients()
    m.forward_prop(b.tensors, "training", b.global_size, 0)
    k._capture(m)
    obj = m.local_objective()
    m.backward_prop(obj)
    cap = gru.kfac_cache[0]
    wih, whh, bih, bhh = gru.ws[0]
    # captured error signals reproduce the layer's own gradients: dW_ih = sum_t g_gi^T x
    g_gi, x = cap["g_gi"].reshape(-1, 3 * H), cap["x"].reshape(-1, I)
    torch.testing.assert_close(g_gi.t() @ x, wih.handle.grad.reshape(3 * H, I), rtol=1e-4, atol=1e-6)
    g_gh, hp = torch.stack(cap["g_gh"], 1).reshape(-1, 3 * H), torch.stack(cap["h_prev"], 1).reshape(-1, H)
    torch.testing.assert_close(g_gh.t() @ hp, whh.handle.grad.reshape(3 * H, H), rtol=1e-4, atol=1e-6)
    raw_w, raw_b = wih.handle.grad.clone().reshape(3 * H, I), bih.handle.grad.clone().reshape(3 * H, 1)
    k._precondition(m, 0, b.global_size)
    a = torch.cat([x, torch.ones(x.shape[0], 1)], 1)
    A = a.t() @ a / a.shape[0]
    Ainv = torch.linalg.inv(A + 0.1 * torch.eye(I + 1))
    g = g_gi * b.global_size
    for gate in range(3):
        gk = g[:, gate * H:(gate + 1) * H]
        Ginv = torch.linalg.inv(gk.t() @ gk / gk.shape[0] + 0.1 * torch.eye(H))
        want = Ginv @ torch.cat([raw_w, raw_b], 1)[gate * H:(gate + 1) * H] @ Ainv
        got = torch.cat([wih.handle.grad.reshape(3 * H, I), bih.handle.grad.reshape(3 * H, 1)], 1)[gate * H:(gate + 1) * H]
        torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-5)
    tr.shutdown()
    # and a whole run
    exp2 = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=11, training_algo=algo), model=model(),
        data_reader=_reader(32, [T * I], "normal", response_dims=[2]), optimizer=lbann.SGD(learn_rate=0.02))
    tr = ExecTrainer(exp2)
    m = tr.build_model(exp2.model)
    first = None
    dc = tr.data_coordinator
    losses = []
    for epoch in range(3):
        dc.start_epoch("training")
        while True:
            bb = dc.next_batch("training")
            if bb is None:
                break
            tr.algorithm.train_mini_batch(tr, m, tr.context(m, "training"), bb, [])
            losses.append(float(m.last_objective))
    tr.shutdown()
    assert all(math.isfinite(v) for v in losses) and sum(losses[-4:]) < sum(losses[:4]), losses


def test_torch_lowering_keeps_registered_user_modules_whole():
    """A user module whose forward cannot be traced (data-dependent branch) is lowered through
    a converter registered for its class; the tracer does not look inside it."""
    import torch.nn as nn
    import lbann_b200.torch as lt
    opts.reset().set("disable_cuda", True)

    class Gate(nn.Module):
        def forward(self, x):
            if float(x.sum()) > 1e30:            # not traceable
                return x
            return torch.relu(x) * 2.0

    @lt.register_opaque(Gate)
    def _gate(m, name, ctx, x):
        return lbann.Scale(lbann.Relu(x, name=name + "_relu"), constant=2.0, name=name)

    net = nn.Sequential(nn.Linear(6, 5), Gate(), nn.Linear(5, 2))
    x = torch.randn(3, 6)
    got = lbann.evaluate(lt.compile(net, input=x)[0], x.numpy())
    torch.testing.assert_close(torch.from_numpy(got), net(x).detach(), rtol=1e-4, atol=1e-5)


def test_kfac_asynchronous_inverses_arrive_one_step_late():
    """With the asynchronous switch an inversion started at step t runs beside the step and is
    installed at step t + 1: after two steps the installed inverses are those of the factors
    after ONE step of the synchronous run (both runs are identical up to there)."""
    from lbann_b200.exec.kfac import KFAC

    def run(steps, asynchronous):
        o = opts.reset()
        o.set("disable_cuda", True)
        if asynchronous:
            o.set("trainer_enable_subgrid_async_comm", True)
        torch.manual_seed(0)
        sgd = lbann.BatchedIterativeOptimizer("sgd", epoch_count=1)
        algo = lbann.KFAC("kfac", sgd, damping_act="1e-2", damping_err="1e-2", kronecker_decay=0.9,
                          update_intervals="1", compute_interval=1)
        exp = lbann.proto.serialize.build_experiment(
            trainer=lbann.Trainer(mini_batch_size=16, random_seed=9, training_algo=algo), model=_mlp(),
            data_reader=_reader(64, [8], "normal", response_dims=[3]),
            optimizer=lbann.SGD(learn_rate=0.05, momentum=0.0))
        tr = ExecTrainer(exp)
        m = tr.build_model(exp.model)
        tr.train(m, num_batches=steps)
        k = tr.algorithm
        assert isinstance(k, KFAC) and k.async_inverses == asynchronous
        inv = {n: (b.Ainv.clone(), b.Ginv.clone()) for n, b in k.blocks.items()}
        obj, _, _ = m.reduce_statistics("training")
        installs, pending = k.async_installs, len(k._pending)
        tr.shutdown()                              # waits for the jobs still running
        assert not k._pending
        return inv, (k.inverses_computed, installs, pending), obj

    sync1, s1, _ = run(1, False)
    async2, a2, _ = run(2, True)
    assert s1 == (4, 0, 0)                         # two blocks, two factors each
    # step 0 inverts in place (nothing to precondition with yet), step 1 starts jobs for both blocks
    assert a2[1] == 0 and a2[2] == 2
    for n in sync1:
        assert torch.allclose(sync1[n][0], async2[n][0], rtol=1e-5, atol=1e-6), n
        assert torch.allclose(sync1[n][1], async2[n][1], rtol=1e-5, atol=1e-6), n
    # longer runs: the late inverses are installed and training still beats plain SGD
    _, a12, obj_async = run(12, True)
    assert a12[1] == 4 * 10 and a12[2] == 2 and a12[0] == 4 * 12
    sgd = lbann.BatchedIterativeOptimizer("sgd", epoch_count=3)
    plain = _fit(sgd)
    assert math.isfinite(obj_async) and obj_async < plain, (plain, obj_async)


def test_kfac_use_interval_switches_between_sgd_and_kfac_by_epoch(capsys):
    """kfac_use_interval "1 2": epoch 0 applies plain SGD gradients (factors are still gathered),
    epoch 1 preconditions, from epoch 2 on K-FAC again (beyond the listed range)."""
    from lbann_b200.exec.kfac import KFAC
    assert KFAC._parse_use_interval("1 2") == [False, True]
    assert KFAC._parse_use_interval("2 4 6") == [False, False, True, True, False, False]
    assert KFAC._parse_use_interval("") == []

    def run(**kw):
        sgd = lbann.BatchedIterativeOptimizer("sgd", epoch_count=1)
        return _fit(lbann.KFAC("kfac", sgd, damping_act="1e-2", damping_err="1e-2", kronecker_decay=0.9,
                               update_intervals="1", compute_interval=1, **kw), epochs=1)

    plain = _fit(lbann.BatchedIterativeOptimizer("sgd", epoch_count=1), epochs=1)
    off = run(kfac_use_interval="1 2", print_time=True, print_matrix_summary=True)   # one epoch: SGD only
    on = run()
    out = capsys.readouterr().out
    assert abs(off - plain) <= 1e-6 * max(1.0, abs(plain)), (off, plain)
    assert on < plain
    assert "(factors only)" in out and "K-FAC fc1: A (9, 9)" in out
