"""Timing of the fused GEMM + collective kernels against their NCCL + GEMM baselines.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m benchmarks.fused_bench [--tokens 8192 --d-model 2048 --ffn 8192]

Shapes follow one transformer FFN: the activations ``[tokens, d_model]`` are sharded by
rows over the ranks (all-gather -> GEMM against a ``[ffn, d_model]`` weight), and the
weight gradient ``dW = dY^T X`` is a product over token slices whose result is scattered by
rows (GEMM -> reduce-scatter).  Every number is the max over ranks of CUDA-event times
(median of ``--iters`` after warm-up, L2 flushed between iterations); rank 0 prints one
JSON line per case with the roofline fraction: target time = the slower of FLOPs at the
measured cuBLAS bf16 peak and bytes over NVLink at the measured 770 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from lbann_b200.ops import native
from lbann_b200.ops.gemm import gemm
from lbann_b200.parallel.comm import LbannComm
from lbann_b200.parallel.fused import FusedGemm
from lbann_b200.parallel.symm import SymmetricGroup

NVLINK_GBS = 770.0


def _peak_tflops() -> float:
    try:
        with open(os.path.join(os.getcwd(), "MEASURED_PEAKS.json")) as f:
            return float(json.load(f).get("bf16_tflops", 1590.0))
    except (OSError, ValueError):
        return 1590.0


def _time(fn, iters, warmup, scratch, pg):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        scratch.fill_(1)
        dist.barrier(group=pg)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, dist.ReduceOp.MAX, group=pg)
    return float(t)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    comm = LbannComm(device=dev)
    g = SymmetricGroup(dev, pg=comm.trainer_group)
    fg = FusedGemm(g)
    P, rank = g.world, g.rank
    dt = torch.bfloat16
    peak = _peak_tflops()
    scratch = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    rows = a.tokens // P
    out = []

    # ---- all-gather -> GEMM:  Y[tokens, ffn] = gather(X)[tokens, d] . W[ffn, d]^T
    xbuf = g.alloc(rows * a.d_model * 2)
    xloc = xbuf.view(dt, rows * a.d_model).view(rows, a.d_model)
    xloc.normal_()
    w = torch.randn(a.ffn, a.d_model, device=dev).to(dt)
    y = torch.empty(a.tokens, a.ffn, dtype=dt, device=dev)
    full = torch.empty(a.tokens, a.d_model, dtype=dt, device=dev)

    def fused_ag():
        fg.allgather_gemm(xbuf, rows, a.d_model, w, sharded="a", dtype=dt, out=y)

    def base_ag():
        dist.all_gather_into_tensor(full, xloc, group=g.pg)
        gemm(full, w, trans_b=True, out=y)

    flops = 2.0 * a.tokens * a.ffn * a.d_model
    link_bytes = (P - 1) * rows * a.d_model * 2
    target = max(flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
    tf, tb = _time(fused_ag, a.iters, a.warmup, scratch, g.pg), _time(base_ag, a.iters, a.warmup, scratch, g.pg)
    out.append({"case": "allgather_gemm", "ranks": P, "shape": [a.tokens, a.ffn, a.d_model],
                "fused_ms": round(tf, 4), "nccl_allgather_plus_gemm_ms": round(tb, 4),
                "target_ms": round(target, 4), "roofline_frac_of_measured": round(target / tf, 3),
                "tflops_per_gpu": round(flops / tf / 1e9, 1)})

    # ---- GEMM -> reduce-scatter:  dW[ffn, d] = sum_r dY_r[rows, ffn]^T . X_r[rows, d], rows of dW scattered
    dy = torch.randn(rows, a.ffn, device=dev).to(dt)
    xr = torch.randn(rows, a.d_model, device=dev).to(dt)
    wrows = a.ffn // P
    obuf = g.alloc(wrows * a.d_model * 4)
    fullw = torch.empty(a.ffn, a.d_model, dtype=torch.float32, device=dev)
    shard = torch.empty(wrows, a.d_model, dtype=torch.float32, device=dev)

    def fused_rs():
        fg.gemm_reduce_scatter(dy, xr, obuf, wrows, trans_a=True, trans_b=True)

    def base_rs():
        gemm(dy, xr, trans_a=True, out=fullw)
        dist.reduce_scatter_tensor(shard, fullw, group=g.pg)

    flops = 2.0 * rows * a.ffn * a.d_model
    link_bytes = (P - 1) * wrows * a.d_model * 4
    target = max(flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
    tf, tb = _time(fused_rs, a.iters, a.warmup, scratch, g.pg), _time(base_rs, a.iters, a.warmup, scratch, g.pg)
    out.append({"case": "gemm_reduce_scatter", "ranks": P, "shape": [a.ffn, a.d_model, rows],
                "fused_ms": round(tf, 4), "gemm_plus_nccl_reduce_scatter_ms": round(tb, 4),
                "target_ms": round(target, 4), "roofline_frac_of_measured": round(target / tf, 3),
                "tflops_per_gpu": round(flops / tf / 1e9, 1)})
    status = native.consume_status(False)
    if rank == 0:
        for o in out:
            o["device_status"] = status
            print(json.dumps(o))
    dist.barrier(group=g.pg)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
