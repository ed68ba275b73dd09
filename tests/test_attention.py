"""Fused attention: the PyTorch formulation on CPU, the tcgen05 kernels on a GPU."""
import math

import pytest
import torch

from lbann_b200.ops import attention as att


def _naive(q, k, v, H, scale, causal):
    B, S, E = q.shape
    D = E // H
    out = torch.zeros(B, S, E, dtype=torch.float64)
    for b in range(B):
        for h in range(H):
            qh, kh, vh = (t[b, :, h * D:(h + 1) * D].double() for t in (q, k, v))
            s = qh @ kh.t() * scale
            if causal:
                s = s + torch.full((S, S), float("-inf"), dtype=torch.float64).triu(1)
            out[b, :, h * D:(h + 1) * D] = torch.softmax(s, -1) @ vh
    return out


def test_reference_attention_matches_per_head_loop():
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 12, 16) for _ in range(3))
    for causal in (False, True):
        y = att.attention(q, k, v, 4, None, causal)
        ref = _naive(q, k, v, 4, 1 / math.sqrt(4), causal)
        assert torch.allclose(y.double(), ref, atol=1e-5)
    qkv = torch.cat([q, k, v], dim=2)
    assert torch.allclose(att.attention_packed(qkv, 4, None, True), att.attention(q, k, v, 4, None, True))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,H,S", [(1, 2, 256), (2, 3, 384)])
def test_fused_attention_forward_backward_vs_fp32(dtype, causal, B, H, S):
    """Outputs and all three gradients of the tcgen05 kernels against fp32 PyTorch attention
    evaluated on the same 16-bit inputs (packed and separate entry points)."""
    torch.manual_seed(1)
    dev = torch.device("cuda")
    E = H * 128
    qkv = (torch.randn(B, S, 3 * E, device=dev) * 0.7).to(dtype).requires_grad_(True)
    assert att.native_ok(qkv[:, :, :E], qkv[:, :, E:2 * E], qkv[:, :, 2 * E:], H, causal)
    scale = 1.0 / math.sqrt(128)
    y = att.attention_packed(qkv, H, scale, causal)
    g = (torch.randn(B, S, E, device=dev) * 0.5).to(dtype)
    y.backward(g)
    ref_in = qkv.detach().float().requires_grad_(True)
    q, k, v = ref_in[:, :, :E], ref_in[:, :, E:2 * E], ref_in[:, :, 2 * E:]
    ref = att.reference_attention(q, k, v, H, scale, causal)
    ref.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert (y.float() - ref).abs().max() <= tol * max(1.0, float(ref.abs().max()))
    gerr = (qkv.grad.float() - ref_in.grad).abs().max()
    assert gerr <= 2 * tol * max(1.0, float(ref_in.grad.abs().max())), float(gerr)
    # separate tensors (cross-attention form), contiguous inputs
    q2, k2, v2 = (t.detach().contiguous().requires_grad_(True) for t in
                  (qkv[:, :, :E], qkv[:, :, E:2 * E], qkv[:, :, 2 * E:]))
    y2 = att.attention(q2, k2, v2, H, scale, causal)
    y2.backward(g)
    assert torch.equal(y2, y)
    assert torch.allclose(torch.cat([q2.grad, k2.grad, v2.grad], 2).float(), qkv.grad.float(), atol=1e-6)
    from lbann_b200.ops import native
    assert native.consume_status(False) == 0


def _gpt_losses(monkeypatch, force):
    import lbann_b200 as lbann
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.models.transformer import construct_gpt_model
    from lbann_b200.utils import options as opts
    if force:
        monkeypatch.setenv("LBANN_FORCE_ATTENTION_FUSION", "1")
    else:
        monkeypatch.delenv("LBANN_FORCE_ATTENTION_FUSION", raising=False)
    o = opts.reset()
    o.set("disable_cuda", True)
    model = construct_gpt_model(vocab_size=64, seq_len=16, d_model=32, num_heads=2, num_layers=2, ffn_dim=64)
    r = lbann.reader_pb2.Reader()
    r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
    r.synth_dimensions, r.num_samples, r.synth_distribution = "17", 8, "randint:64"
    dr = lbann.reader_pb2.DataReader()
    dr.reader.append(r)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=4, random_seed=1), model=model, data_reader=dr,
        optimizer=lbann.SGD(learn_rate=0.1))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    fused = [l.name for l in m.layers if getattr(l, "attention", None)]
    dead = sum(1 for l in m.layers if getattr(l, "dead", False))
    dc = tr.data_coordinator
    dc.start_epoch("training")
    losses = []
    for _ in range(2):
        b = dc.next_batch("training")
        m.train_step(b.tensors, b.global_size)
        losses.append(float(m.last_objective))
    tr.shutdown()
    return losses, fused, dead


def test_attention_subgraph_is_replaced_by_one_call(monkeypatch):
    """The executor recognises the front end's attention sub-graph (reshape / permute / two
    MatMuls / scale / mask / softmax) and replaces it with one attention call per block; the
    training losses are the same as layer by layer."""
    plain = _gpt_losses(monkeypatch, False)
    fused = _gpt_losses(monkeypatch, True)
    assert not plain[1] and len(fused[1]) == 2 and fused[2] >= 2 * 12
    for a, b in zip(plain[0], fused[0]):
        assert abs(a - b) < 1e-4
