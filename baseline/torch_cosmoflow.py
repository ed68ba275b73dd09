"""Comparison arm: the same CosmoFlow configuration on the library stack the reference sits
on (cuDNN convolutions / cuBLAS GEMMs through torch.nn, NCCL through DistributedDataParallel).
None of this framework's kernels or engine are used here.  With several GPUs the global
mini-batch of 8 is split over ranks (sample parallelism), the only decomposition the plain
library stack offers."""
from __future__ import annotations

import json
import os
import time

import torch
import torch.nn as nn


def build(width):
    chans = [4, 32, 64, 128, 256, 256]
    layers = []
    for i in range(5):
        layers += [nn.Conv3d(chans[i], chans[i + 1], 3, padding=1, bias=False), nn.LeakyReLU(0.3),
                   nn.MaxPool3d(2)]
    feat = 256 * (width // 32) ** 3
    layers += [nn.Flatten(), nn.Linear(feat, 2048), nn.LeakyReLU(0.3), nn.Linear(2048, 256),
               nn.LeakyReLU(0.3), nn.Linear(256, 4)]
    return nn.Sequential(*layers)


def measure_torch(steps, warm, global_batch, width):
    """The comparison arm inside an already initialised process group (called by bench.py
    after its own measurement): same model, cuDNN autotuning on, DistributedDataParallel over
    NCCL when there are several ranks.  Returns a dict (device-timed and end to end)."""
    import torch.distributed as dist
    world = dist.get_world_size() if dist.is_initialized() else 1
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.backends.cudnn.benchmark = True           # the reference autotunes (cudnnFind*Ex)
    torch.manual_seed(1)
    model = build(width).to(dev).to(memory_format=torch.channels_last_3d)
    if world > 1:
        model = nn.parallel.DistributedDataParallel(model, device_ids=[local])
    opt = torch.optim.Adam(model.parameters(), lr=1e-3, betas=(0.9, 0.99), eps=1e-8, fused=True)
    scaler = torch.amp.GradScaler("cuda", init_scale=128.0)
    nb = max(global_batch // world, 1)
    batches = []
    for i in range(2):
        x = torch.randn(nb, 4, width, width, width, device=dev).exp().half().contiguous(
            memory_format=torch.channels_last_3d)
        batches.append((x, torch.rand(nb, 4, device=dev) * 2 - 1))

    def step(x, y):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.float16):
            out = model(x)
        loss = nn.functional.mse_loss(out.float(), y)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        return loss

    for i in range(max(warm, 3) + 2):
        step(*batches[i % 2])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = step(*batches[i % 2])
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    hx = [b[0].cpu().pin_memory() for b in batches]
    hy = [b[1].cpu().pin_memory() for b in batches]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(steps):
        x = hx[i % 2].to(dev, non_blocking=True)
        y = hy[i % 2].to(dev, non_blocking=True)
        float(step(x, y))
    torch.cuda.synchronize()
    e2e = torch.tensor([(time.perf_counter() - t0) * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(ms, dist.ReduceOp.MAX)
        dist.all_reduce(e2e, dist.ReduceOp.MAX)
    ms, e2e = float(ms), float(e2e)
    out = {"impl": "torch + cuDNN (benchmark mode) + NCCL DDP", "n_gpus": world,
           "global_batch": nb * world, "ms_per_step": round(ms / steps, 4),
           "value": round(nb * world * steps / (ms / 1e3), 3), "unit": "samples/s",
           "e2e": {"value": round(nb * world * steps / (e2e / 1e3), 3), "unit": "samples/s"},
           "final_loss": float(loss), "loss_scale": float(scaler.get_scale()),
           "parallelism": f"ddp x{world} (sample parallel)" if world > 1 else "single GPU"}
    del model, opt, batches, hx, hy
    torch.cuda.empty_cache()
    return out


def run(args, global_batch, width, baseline, ClockSampler):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1)
    torch.backends.cudnn.benchmark = True           # the reference autotunes (cudnnFind*Ex)
    model = build(width).to(dev).to(memory_format=torch.channels_last_3d)
    if world > 1:
        model = nn.parallel.DistributedDataParallel(model, device_ids=[local])
    opt = torch.optim.Adam(model.parameters(), lr=1e-3, betas=(0.9, 0.99), eps=1e-8, fused=True)
    scaler = torch.amp.GradScaler("cuda", init_scale=128.0)
    nb = max(global_batch // world, 1)
    batches = []
    for i in range(2):
        x = torch.randn(nb, 4, width, width, width, device=dev).exp().half().contiguous(
            memory_format=torch.channels_last_3d)
        y = (torch.rand(nb, 4, device=dev) * 2 - 1)
        batches.append((x, y))

    def step(x, y):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.float16):
            out = model(x)
        loss = nn.functional.mse_loss(out.float(), y)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        return loss

    warm, steps = max(args.warmup, 3), args.steps
    for i in range(warm):
        step(*batches[i % 2])
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = step(*batches[i % 2])
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        torch.distributed.all_reduce(ms, torch.distributed.ReduceOp.MAX)
    # end to end: pinned host batch -> device and loss read-back every step
    hx = [b[0].cpu().pin_memory() for b in batches]
    hy = [b[1].cpu().pin_memory() for b in batches]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(steps):
        x = hx[i % 2].to(dev, non_blocking=True)
        y = hy[i % 2].to(dev, non_blocking=True)
        float(step(x, y))
    torch.cuda.synchronize()
    e2e_ms = torch.tensor([(time.perf_counter() - t0) * 1e3], device=dev)
    if world > 1:
        torch.distributed.all_reduce(e2e_ms, torch.distributed.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        ms, e2e_ms = float(ms), float(e2e_ms)
        val = nb * world * steps / (ms / 1e3)
        print(json.dumps({
            "metric": "CosmoFlow distconv training throughput", "value": round(val, 3),
            "unit": "samples/s", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": round(ms / steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(val / baseline, 3), "dtype": "fp16", "data": "synthetic",
            "impl": "torch+cudnn+nccl",
            "config": {"model": "CosmoFlow 128^3 (same layers)", "global_batch": nb * world,
                       "parallelism": f"ddp x{world}" if world > 1 else "single GPU"},
            "e2e": {"value": round(nb * world * steps / (e2e_ms / 1e3), 3), "unit": "samples/s",
                    "h2d_bytes_per_step": int(hx[0].numel() * 2 + hy[0].numel() * 4),
                    "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "clocks": clocks}))
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0
