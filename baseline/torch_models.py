"""Comparison arms for the ResNet-50 and GPT entries of bench.py: the same architectures on
torch.nn (cuDNN convolutions in autotune mode, cuBLAS GEMMs, SDPA attention, fused
optimizers) with DistributedDataParallel over NCCL.  None of this framework's kernels or
engine are used here.  Called from bench.py inside its process group."""
from __future__ import annotations

import os
import time

import torch
import torch.nn as nn
import torch.nn.functional as F


def resnet50():
    def bottleneck(cin, mid, stride):
        out = 4 * mid
        body = nn.Sequential(nn.Conv2d(cin, mid, 1, bias=False), nn.BatchNorm2d(mid), nn.ReLU(True),
                             nn.Conv2d(mid, mid, 3, stride, 1, bias=False), nn.BatchNorm2d(mid), nn.ReLU(True),
                             nn.Conv2d(mid, out, 1, bias=False), nn.BatchNorm2d(out))
        short = None if (stride == 1 and cin == out) else nn.Sequential(
            nn.Conv2d(cin, out, 1, stride, bias=False), nn.BatchNorm2d(out))
        return body, short

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.stem = nn.Sequential(nn.Conv2d(3, 64, 7, 2, 3, bias=False), nn.BatchNorm2d(64),
                                      nn.ReLU(True), nn.MaxPool2d(3, 2, 1))
            self.bodies, self.shorts = nn.ModuleList(), nn.ModuleList()
            cin = 64
            for stage, (n, mid) in enumerate(zip((3, 4, 6, 3), (64, 128, 256, 512))):
                for i in range(n):
                    b, s = bottleneck(cin, mid, 2 if (i == 0 and stage > 0) else 1)
                    self.bodies.append(b)
                    self.shorts.append(s if s is not None else nn.Identity())
                    cin = 4 * mid
            self.fc = nn.Linear(2048, 1000, bias=False)

        def forward(self, x):
            x = self.stem(x)
            for b, s in zip(self.bodies, self.shorts):
                x = F.relu(b(x) + s(x))
            return self.fc(x.mean((2, 3)))

    return Net()


class GPT(nn.Module):
    def __init__(self, layers, d_model=2048, heads=16, seq=2048, vocab=50304):
        super().__init__()
        layer = nn.TransformerEncoderLayer(d_model, heads, 4 * d_model, 0.0, "gelu", batch_first=True,
                                           norm_first=True)
        self.seq = seq
        self.emb = nn.Embedding(vocab, d_model)
        self.pos = nn.Parameter(torch.zeros(seq, d_model))
        self.blocks = nn.TransformerEncoder(layer, layers, enable_nested_tensor=False)
        self.norm = nn.LayerNorm(d_model)
        self.head = nn.Linear(d_model, vocab, bias=False)

    def forward(self, t):
        x = self.emb(t) + self.pos
        mask = nn.Transformer.generate_square_subsequent_mask(self.seq, device=t.device)
        return self.head(self.norm(self.blocks(x, mask=mask, is_causal=True)))


def measure_torch_model(name, args, world, rank, local_rank):
    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    torch.backends.cudnn.benchmark = True
    torch.manual_seed(0)
    if name == "resnet50":
        batch = args.resnet_batch
        net = resnet50().to(dev).to(memory_format=torch.channels_last)
        opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
        x = torch.randn(batch, 3, 224, 224, device=dev).to(memory_format=torch.channels_last)
        y = torch.randint(0, 1000, (batch,), device=dev)
        steps, unit, per_step = max(min(args.steps, 10), 3), "images/s", batch * world
        host = (x.cpu().pin_memory(), y.cpu().pin_memory())

        def fwd(net, x, y):
            with torch.autocast("cuda", torch.bfloat16):
                return F.cross_entropy(net(x), y)
    else:
        batch, seq, vocab = args.gpt_batch, 2048, 50304
        net = GPT(args.gpt_layers, seq=seq, vocab=vocab).to(dev)
        opt = torch.optim.Adam(net.parameters(), lr=3e-4, betas=(0.9, 0.95), fused=True)
        tok = torch.randint(0, vocab, (batch, seq + 1), device=dev)
        x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        steps, unit, per_step = max(min(args.steps, 5), 2), "tokens/s", batch * world * seq
        host = (x.cpu().pin_memory(), y.cpu().pin_memory())

        def fwd(net, x, y):
            with torch.autocast("cuda", torch.bfloat16):
                logits = net(x)
            return F.cross_entropy(logits.reshape(-1, vocab).float(), y.reshape(-1))
    if world > 1:
        net = nn.parallel.DistributedDataParallel(net, device_ids=[local_rank])

    def step(x, y):
        opt.zero_grad(set_to_none=True)
        loss = fwd(net, x, y)
        loss.backward()
        opt.step()
        return loss

    for _ in range(4):
        step(x, y)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step(x, y)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        float(step(host[0].to(dev, non_blocking=True), host[1].to(dev, non_blocking=True)))
    torch.cuda.synchronize()
    e2e = torch.tensor([(time.perf_counter() - t0) * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(ms, dist.ReduceOp.MAX)
        dist.all_reduce(e2e, dist.ReduceOp.MAX)
    ms, e2e = float(ms) / steps, float(e2e) / steps
    out = {"impl": "torch (cuDNN autotuned / cuBLAS / SDPA) + NCCL DDP", "n_gpus": world,
           "ms_per_step": round(ms, 3), "value": round(per_step / ms * 1e3, 2), "unit": unit,
           "e2e": {"value": round(per_step / e2e * 1e3, 2), "unit": unit, "ms_per_step": round(e2e, 3)},
           "final_loss": float(loss), "steps": steps}
    del net, opt
    torch.cuda.empty_cache()
    return out
