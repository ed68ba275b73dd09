#!/usr/bin/env python
"""Secondary training-throughput benchmarks: ResNet-50 (data-parallel) and a GPT decoder.

    python bench_models.py --model resnet50 --batch 64 --steps 20 --warmup 5
    python bench_models.py --model gpt --layers 4 --batch 2 --steps 10
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        bench_models.py --model resnet50 --batch 64          # per-GPU batch, data parallel

Synthetic data, random-initialised weights, bf16 compute with fp32 master weights.  The
timed region is ``steps`` training steps (forward, backward, gradient all-reduce, fused
optimizer) on mini-batches that already sit in device memory, bracketed by CUDA events and
a barrier; the result is the max over ranks.  ``--impl torch`` runs the same architecture
through torch.nn + cuDNN / cuBLAS for reference.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _build(lbann, args, world):
    if args.model == "resnet50":
        from lbann_b200.models import ResNet50, construct_classifier
        from lbann_b200.models.cosmoflow import synthetic_reader  # noqa: F401  (same reader class)
        model = construct_classifier(ResNet50(1000, bn_statistics_group_size=1), 1000)
        r = lbann.reader_pb2.Reader()
        r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
        r.synth_dimensions = f"3 {args.image} {args.image}"
        r.num_samples = 2 * args.batch * world
        r.num_labels = 1000
        r.synth_pool_size = 2 * args.batch * world
        opt = lbann.SGD(learn_rate=0.1, momentum=0.9)
    elif args.model == "unet3d":
        # 3D U-Net with batch norm, per-voxel 3-class cross-entropy; with several ranks the
        # depth dimension is split over them (strong scaling of one global mini-batch)
        from lbann_b200.models import construct_unet3d_model
        # --height-groups H: a (world / H) x H grid over depth and height instead of depth only
        hg, wg = max(1, args.height_groups), max(1, args.width_groups)
        ps = lbann.get_parallel_strategy_args(depth_groups=world // (hg * wg), height_groups=hg,
                                              width_groups=wg) if world > 1 else None
        model = construct_unet3d_model(num_classes=3, base_channels=32, levels=4, parallel_strategy=ps)
        v = args.volume
        r = lbann.reader_pb2.Reader()
        r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
        r.synth_dimensions = f"1 {v} {v} {v}"
        r.synth_response_dimensions = f"{v} {v} {v}"
        r.synth_distribution = "samples:normal responses:randint:3"
        r.num_samples = 2 * args.batch
        r.synth_pool_size = 2 * args.batch
        opt = lbann.Adam(learn_rate=1e-3, beta1=0.9, beta2=0.99, eps=1e-8)
        dr = lbann.reader_pb2.DataReader()
        dr.reader.append(r)
        return lbann.proto.serialize.build_experiment(
            trainer=lbann.Trainer(mini_batch_size=args.batch, random_seed=1), model=model,
            data_reader=dr, optimizer=opt)
    else:
        from lbann_b200.models.transformer import construct_gpt_model
        model = construct_gpt_model(vocab_size=args.vocab, seq_len=args.seq, d_model=args.d_model,
                                    num_heads=args.heads, num_layers=args.layers, ffn_dim=4 * args.d_model)
        r = lbann.reader_pb2.Reader()
        r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
        r.synth_dimensions = str(args.seq + 1)
        r.num_samples = 2 * args.batch * world
        r.synth_distribution = f"randint:{args.vocab}"
        r.synth_pool_size = 2 * args.batch * world
        opt = lbann.Adam(learn_rate=3e-4, beta1=0.9, beta2=0.95, eps=1e-8)
    dr = lbann.reader_pb2.DataReader()
    dr.reader.append(r)
    return lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=args.batch * world, random_seed=1), model=model,
        data_reader=dr, optimizer=opt)


def ours(args):
    import lbann_b200 as lbann
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.ops import native
    from lbann_b200.utils import options as opts
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    o = opts.reset()
    o.set("default_dtype", "bf16")
    if args.graph:
        o.set("use_cuda_graph", True)
    exp = _build(lbann, args, world)
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dev = tr.device
    dc = tr.data_coordinator
    dc.start_epoch("training")
    batches = [dc.next_batch("training"), dc.next_batch("training")]
    for i in range(max(args.warmup, 3) + (4 if args.graph else 0)):     # + ordinary steps and capture
        b = batches[i % 2]
        m.train_step(b.tensors, b.global_size)
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    n0 = native.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        b = batches[i % 2]
        m.train_step(b.tensors, b.global_size)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        torch.distributed.all_reduce(ms, torch.distributed.ReduceOp.MAX)
    ms = float(ms) / args.steps
    status = native.consume_status(False)
    loss = float(m.last_objective)
    if rank == 0:
        gb = args.batch if args.model == "unet3d" else args.batch * world
        out = {"model": args.model, "impl": "lbann_b200", "n_gpus": world, "global_batch": gb,
               "ms_per_step": round(ms, 3), "samples_per_s": round(gb / ms * 1e3, 2), "dtype": "bf16",
               "gpu_launches": native.launches() - n0, "loss": loss, "device_status": status,
               "cuda_graph": bool(getattr(m, "_graph_mode", False))}
        if args.model == "unet3d" and world > 1:
            hg, wg = max(1, args.height_groups), max(1, args.width_groups)
            out["parallelism"] = f"distconv depth x{world // (hg * wg)}" + (f" height x{hg}" if hg > 1 else "") + \
                (f" width x{wg}" if wg > 1 else "")
        if args.model == "gpt":
            out["tokens_per_s"] = round(gb * args.seq / ms * 1e3, 1)
            out["config"] = {"layers": args.layers, "d_model": args.d_model, "heads": args.heads,
                             "seq": args.seq, "vocab": args.vocab}
        print(json.dumps(out))
    tr.shutdown()


def torch_arm(args):
    """The same architectures through torch.nn (cuDNN / cuBLAS / SDPA), bf16 autocast."""
    import torch.nn as nn
    import torch.nn.functional as F
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    if args.model == "resnet50":
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

        net = Net().to(dev).to(memory_format=torch.channels_last)
        opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
        x = torch.randn(args.batch, 3, args.image, args.image, device=dev).to(memory_format=torch.channels_last)
        y = torch.randint(0, 1000, (args.batch,), device=dev)

        def step():
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", torch.bfloat16):
                loss = F.cross_entropy(net(x), y)
            loss.backward()
            opt.step()
            return loss
    else:
        layer = nn.TransformerEncoderLayer(args.d_model, args.heads, 4 * args.d_model, 0.0, "gelu",
                                           batch_first=True, norm_first=True)

        class GPT(nn.Module):
            def __init__(self):
                super().__init__()
                self.emb = nn.Embedding(args.vocab, args.d_model)
                self.pos = nn.Parameter(torch.zeros(args.seq, args.d_model))
                self.blocks = nn.TransformerEncoder(layer, args.layers, enable_nested_tensor=False)
                self.norm = nn.LayerNorm(args.d_model)
                self.head = nn.Linear(args.d_model, args.vocab, bias=False)

            def forward(self, t):
                x = self.emb(t) + self.pos
                mask = nn.Transformer.generate_square_subsequent_mask(args.seq, device=t.device)
                return self.head(self.norm(self.blocks(x, mask=mask, is_causal=True)))

        net = GPT().to(dev)
        opt = torch.optim.Adam(net.parameters(), lr=3e-4, betas=(0.9, 0.95), fused=True)
        tok = torch.randint(0, args.vocab, (args.batch, args.seq + 1), device=dev)

        def step():
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", torch.bfloat16):
                logits = net(tok[:, :-1])
                loss = F.cross_entropy(logits.reshape(-1, args.vocab).float(), tok[:, 1:].reshape(-1))
            loss.backward()
            opt.step()
            return loss

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    out = {"model": args.model, "impl": "torch (cuDNN / cuBLAS / SDPA)", "n_gpus": 1, "global_batch": args.batch,
           "ms_per_step": round(ms, 3), "samples_per_s": round(args.batch / ms * 1e3, 2), "dtype": "bf16",
           "loss": float(loss)}
    if args.model == "gpt":
        out["tokens_per_s"] = round(args.batch * args.seq / ms * 1e3, 1)
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "gpt", "unet3d"])
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    ap.add_argument("--batch", type=int, default=64, help="per-GPU mini-batch")
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--volume", type=int, default=128, help="edge of the U-Net input volume")
    ap.add_argument("--height-groups", type=int, default=1,
                    help="U-Net: ranks along height (the rest of the ranks split depth)")
    ap.add_argument("--width-groups", type=int, default=1, help="U-Net: ranks along width")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--graph", action="store_true", help="capture the step as a CUDA graph and replay it")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_models.py needs a GPU")
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    (ours if args.impl == "ours" else torch_arm)(args)


if __name__ == "__main__":
    main()
