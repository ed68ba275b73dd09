"""Loss trajectories against plain PyTorch restatements ("twins") of the same architectures
that start from the SAME weights and see the same mini-batches: ten SGD steps of the small
CosmoFlow and of a two-layer GPT must agree step by step (fp32 on CPU)."""
import math

import torch
import torch.nn.functional as F

import lbann_b200 as lbann
from lbann_b200.exec.trainer import ExecTrainer
from lbann_b200.utils import options as opts
from test_models_cpu import _reader

STEPS = 10


def _framework_run(model, reader, mb, lr):
    o = opts.reset()
    o.set("disable_cuda", True)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=mb, random_seed=5), model=model, data_reader=reader,
        optimizer=lbann.SGD(learn_rate=lr, momentum=0.9))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    start = {w.name: w.values.detach().clone() for w in m.weights}
    dc = tr.data_coordinator
    dc.start_epoch("training")
    batches, losses = [], []
    for _ in range(STEPS):
        b = dc.next_batch("training")
        if b is None:
            dc.start_epoch("training")
            b = dc.next_batch("training")
        batches.append({k: v.clone() for k, v in b.tensors.items()})
        m.train_step(b.tensors, b.global_size)
        losses.append(float(m.last_objective))
    tr.shutdown()
    return start, batches, losses


def _sgd(params, lr, momentum=0.9):
    return torch.optim.SGD(params, lr=lr, momentum=momentum)


def test_cosmoflow_trajectory_equals_a_pytorch_twin():
    from lbann_b200.models.cosmoflow import construct_cosmoflow_model
    torch.manual_seed(0)
    channels, fcs = (4, 8, 8), (16, 8)
    model = construct_cosmoflow_model(16, 2, 3, num_epochs=1, channels=channels, pool_mode="max", conv_bias=True,
                                      fc_sizes=fcs)
    start, batches, losses = _framework_run(model, _reader(16, [2, 16, 16, 16], "normal", response_dims=[3]), 4, 0.01)
    conv_w = sorted(k for k in start if k.endswith("_kernel"))
    conv_b = {k[:-len("_kernel")]: k[:-len("_kernel")] + "_bias" for k in conv_w}
    fc_w = sorted(k for k in start if k.endswith("_matrix"))
    p = {k: v.clone().requires_grad_(True) for k, v in start.items()}
    opt = _sgd(list(p.values()), 0.01)
    slope = 0.3                                           # the model's leaky-ReLU slope
    twin = []
    for b in batches:
        h = b["samples"].reshape(-1, 2, 16, 16, 16)
        for k in conv_w:
            h = F.max_pool3d(F.leaky_relu(F.conv3d(h, p[k], p.get(conv_b[k[:-len("_kernel")]]), padding=1), slope), 2)
        h = h.flatten(1)
        for i, k in enumerate(fc_w):
            h = F.linear(h, p[k], p.get(k[:-len("_matrix")] + "_bias"))
            if i < len(fc_w) - 1:
                h = F.leaky_relu(h, slope)
        loss = F.mse_loss(h, b["responses"].reshape(h.shape))
        twin.append(float(loss.detach()))
        opt.zero_grad()
        loss.backward()
        opt.step()
    for a, c in zip(losses, twin):
        assert abs(a - c) <= 1e-4 * max(1.0, abs(c)), (losses, twin)
    assert twin[-1] != twin[0]


def test_gpt_trajectory_equals_a_pytorch_twin():
    from lbann_b200.models.transformer import construct_gpt_model
    torch.manual_seed(0)
    V, S, E, H, NL, FF = 24, 8, 16, 2, 2, 32
    model = construct_gpt_model(vocab_size=V, seq_len=S, d_model=E, num_heads=H, num_layers=NL, ffn_dim=FF)
    start, batches, losses = _framework_run(model, _reader(16, [S + 1], f"randint:{V}"), 4, 0.05)
    p = {k: v.clone().requires_grad_(not k.endswith("causal_values")) for k, v in start.items()}
    opt = _sgd([v for v in p.values() if v.requires_grad], 0.05)
    twin = []
    for b in batches:
        tok = b["samples"].reshape(-1, S + 1).long()
        x = p["gpt_token_embeddings"][tok[:, :S]] + p["gpt_positions_positions"]
        mask = p["gpt_causal_values"].reshape(S, S)
        for l in range(NL):
            n = f"gpt_block{l}_"
            h = F.layer_norm(x, (E,), p[n + "norm1_weight"], p[n + "norm1_bias"], 1e-5)
            qkv = F.linear(h, p[n + "attention_qkv_matrix"], p[n + "attention_qkv_bias"])
            q, k, v = (t.reshape(-1, S, H, E // H).transpose(1, 2) for t in qkv.split(E, dim=-1))
            att = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(E // H) + mask, dim=-1) @ v
            x = x + F.linear(att.transpose(1, 2).reshape(-1, S, E), p[n + "attention_output_matrix"],
                             p[n + "attention_output_bias"])
            h = F.layer_norm(x, (E,), p[n + "norm2_weight"], p[n + "norm2_bias"], 1e-5)
            x = x + F.linear(F.gelu(F.linear(h, p[n + "fc1_matrix"], p[n + "fc1_bias"])), p[n + "fc2_matrix"],
                             p[n + "fc2_bias"])
        x = F.layer_norm(x, (E,), p["gpt_final_norm_weight"], p["gpt_final_norm_bias"], 1e-5)
        logits = F.linear(x, p["gpt_lm_head"])
        loss = F.cross_entropy(logits.reshape(-1, V), tok[:, 1:].reshape(-1), reduction="sum") / (tok.shape[0] * S)
        twin.append(float(loss.detach()))
        opt.zero_grad()
        loss.backward()
        opt.step()
    for a, c in zip(losses, twin):
        assert abs(a - c) <= 2e-4 * max(1.0, abs(c)), (losses, twin)
    assert twin[-1] < twin[0]


def test_resnet18_trajectory_equals_a_pytorch_twin():
    from lbann_b200.models.resnet import ResNet18, construct_classifier
    torch.manual_seed(0)
    net = ResNet18(10, zero_init_residual=False, name="rn", width=0.125)          # 8/16/32/64 channels
    model = construct_classifier(net, 10)
    start, batches, losses = _framework_run(model, _reader(32, [3, 64, 64], "normal", label_classes=10), 8, 0.005)
    trainable = [k for k in start if not (k.endswith("running_mean") or k.endswith("running_variance"))]
    p = {k: start[k].clone().requires_grad_(True) for k in trainable}
    assert any(k.endswith("_bn_scale") for k in p) and "rn_fc_matrix" in p, sorted(start)
    opt = _sgd(list(p.values()), 0.005)

    def cbr(x, n, stride, pad, relu):
        y = F.conv2d(x, p[n + "_conv_kernel"], None, stride=stride, padding=pad)
        # the reference's batch norm: Bessel-corrected batch variance, clamped at epsilon
        cnt = y.numel() / y.shape[1]
        mean = y.mean(dim=(0, 2, 3), keepdim=True)
        var = (y.var(dim=(0, 2, 3), keepdim=True, unbiased=False) * cnt / (cnt - 1)).clamp(min=1e-5)
        y = (y - mean) / torch.sqrt(var + 1e-5) * p[n + "_bn_scale"].view(1, -1, 1, 1) + p[n + "_bn_bias"].view(1, -1, 1, 1)
        return F.relu(y) if relu else y

    twin = []
    for b in batches:
        x = b["samples"].reshape(-1, 3, 64, 64)
        x = F.max_pool2d(cbr(x, "rn_conv1", 2, 3, True), 3, 2, 1)
        cin = 8
        for stage, ch in enumerate((8, 16, 32, 64)):
            for i in range(2):
                n = f"rn_layer{stage + 1}_block{i}"
                down = i == 0 and stage > 0
                y = cbr(cbr(x, n + "_branch2a", 2 if down else 1, 1, True), n + "_branch2b", 1, 1, False)
                s = cbr(x, n + "_branch1", 2 if down else 1, 0, False) if (down or cin != ch) else x
                x, cin = F.relu(y + s), ch
        logits = F.linear(x.mean(dim=(2, 3)), p["rn_fc_matrix"])
        loss = F.cross_entropy(logits, b["labels"].reshape(logits.shape).argmax(dim=1))
        twin.append(float(loss.detach()))
        opt.zero_grad()
        loss.backward()
        opt.step()
    for a, c in zip(losses, twin):
        assert abs(a - c) <= 5e-4 * max(1.0, abs(c)), (losses, twin)
    assert twin[-1] != twin[0]
