"""Single-kernel timing harness: ``python -m benchmarks.microbench <case> [options]``.

Each case runs one native kernel (or one layer's forward / backward pair) on a
stated shape, times it with CUDA events on the launching stream after warm-up,
writes a buffer larger than L2 between timed iterations, and prints one JSON
line with the algorithmic FLOPs and bytes, the achieved rates and -- when a
``MEASURED_PEAKS.json`` sits in the working directory -- the fractions of the
measured copy bandwidth and cuBLAS bf16 throughput.  The same command line is
what a profiler capture of that kernel wraps.

Cases: ``gemm``, ``gemm_comm`` (fused GEMM + collective kernel in a one-GPU layout), ``conv`` (forward and, with ``--bwd``, data and filter
gradients; the first-layer kernels are chosen automatically for <= 8 input
channels), ``pool``, ``optimizer``, ``linear_wgrad`` (weight gradient of a fully-connected
layer; ``--m`` rows of mini-batch, ``--n`` outputs, ``--k`` inputs), ``bn`` (batch norm + ReLU, ``--batch --cin --size``).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from lbann_b200.ops import native


def _peaks():
    try:
        with open(os.path.join(os.getcwd(), "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", 0.0)), float(d.get("bf16_tflops", 0.0))
    except (OSError, ValueError):
        return 0.0, 0.0


class _Timer:
    def __init__(self, iters: int, warmup: int, flush: bool = True):
        self.iters, self.warmup = iters, warmup
        self.scratch = torch.empty(192 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def run(self, fn):
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(self.iters):
            if self.scratch is not None:
                self.scratch.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        times.sort()
        return times[len(times) // 2], times[0]


def _report(name, shape, ms, ms_min, flops, nbytes):
    hbm, tf = _peaks()
    out = {"case": name, "shape": shape, "ms_median": round(ms, 4), "ms_min": round(ms_min, 4),
           "tflops": round(flops / ms / 1e9, 2), "gbs": round(nbytes / ms / 1e6, 1)}
    if hbm > 0:
        out["frac_hbm_of_measured"] = round(out["gbs"] / hbm, 3)
    if tf > 0:
        out["frac_bf16_of_measured"] = round(out["tflops"] / tf, 3)
    print(json.dumps(out))
    return out


def _dtype(name):
    return {"fp16": torch.float16, "bf16": torch.bfloat16}[name]


def case_gemm(a, timer):
    from lbann_b200.ops.gemm import gemm
    dt = _dtype(a.dtype)
    A = torch.randn(a.m, a.k, device="cuda", dtype=dt)
    B = torch.randn(a.n, a.k, device="cuda", dtype=dt)
    C = torch.empty(a.m, a.n, device="cuda", dtype=dt)
    ms, mn = timer.run(lambda: gemm(A, B, trans_b=True, out=C))
    return _report("gemm", [a.m, a.n, a.k], ms, mn, 2.0 * a.m * a.n * a.k,
                   2.0 * (a.m * a.k + a.n * a.k + a.m * a.n))


def case_conv(a, timer):
    from lbann_b200.ops import nn
    dt = _dtype(a.dtype)
    N, C, K, S, ks = a.batch, a.cin, a.cout, a.size, a.ksize
    x = torch.randn(N, S, S, S, C, device="cuda", dtype=dt).permute(0, 4, 1, 2, 3)
    x.requires_grad_(a.bwd and C > 8)
    w = torch.randn(K, C, ks, ks, ks, device="cuda") * 0.05
    wh = nn.WeightHandle(w.requires_grad_(True), torch.zeros_like(w))
    pad = (ks - 1) // 2
    px = float(N) * S ** 3
    flops = 2.0 * px * K * C * ks ** 3
    fwd_bytes = 2.0 * px * (max(C, 8) + K)
    out = []

    act = native.ACT_LEAKY if a.act else native.ACT_NONE

    def fwd():
        # --pool: the 2x2x2 max pooling behind a first-layer convolution, as a second kernel
        # ("separate") or inside the convolution kernel ("fused")
        fuse = nn.PoolFusion() if a.pool == "fused" else None
        y = nn.convolution(x, wh, None, (ks,) * 3, (pad,) * 3, (1,) * 3, (1,) * 3, act=act, act_param=0.3,
                           skip_act_grad=a.pool != "none", fuse_pool=fuse)
        if a.pool == "separate" or (fuse is not None and not fuse.done):
            y = nn.pooling(y, 2, 0, 2, "max", act, 0.3)
        return y

    ms, mn = timer.run(fwd)
    if a.pool != "none":
        fwd_bytes = 2.0 * px * (max(C, 8) + K / 8) + px * K / 8
    out.append(_report("conv_fwd" if a.pool == "none" else f"conv_fwd+pool({a.pool})",
                       [N, C, K, S, ks], ms, mn, flops, fwd_bytes))
    if a.bwd:
        y = fwd()
        dy = torch.randn_like(y)

        def bwd():
            y.backward(dy, retain_graph=True)

        ms, mn = timer.run(bwd)
        nmm = 2 if x.requires_grad else 1
        out.append(_report("conv_bwd(dgrad+wgrad)" if nmm == 2 else "conv_bwd(wgrad)",
                           [N, C, K, S, ks], ms, mn, nmm * flops, nmm * fwd_bytes))
    return out


def case_pool(a, timer):
    from lbann_b200.ops import nn
    dt = _dtype(a.dtype)
    N, C, S = a.batch, a.cin, a.size
    x = torch.randn(N, S, S, S, C, device="cuda", dtype=dt).permute(0, 4, 1, 2, 3)
    x.requires_grad_(True)
    px = float(N) * S ** 3 * C
    ms, mn = timer.run(lambda: nn.pooling(x, 2, 0, 2, "max"))
    out = [_report("pool_fwd", [N, C, S], ms, mn, 0.0, 2.0 * px * (1 + 1 / 8))]
    if a.bwd:
        y = nn.pooling(x, 2, 0, 2, "max")
        dy = torch.randn_like(y)
        ms, mn = timer.run(lambda: y.backward(dy, retain_graph=True))
        out.append(_report("pool_bwd", [N, C, S], ms, mn, 0.0, 2.0 * px * (2 + 1 / 8)))
    return out


def case_gemm_comm(a, timer):
    """The fused GEMM + collective kernel on ONE GPU: both "ranks" of a two-rank layout are
    buffers of this device, so the copying CTAs, the per-block flags and the reduce-scatter
    epilogue all run (their traffic stays in local memory instead of crossing NVLink).
    This is the form a profiler can capture; multi-GPU timings come from
    ``python -m benchmarks.fused_bench``."""
    import ctypes
    from lbann_b200.parallel import fused
    lib = fused._lib()
    dt = _dtype(a.dtype)
    P = 2
    M, N, K = a.m, a.n, a.k
    rows = M // P
    c_void_p = ctypes.c_void_p
    out = []
    # all-gather -> GEMM with in-kernel staging: A = two row shards
    shards = [torch.randn(rows, K, device="cuda", dtype=dt) for _ in range(P)]
    W = torch.randn(N, K, device="cuda", dtype=dt)
    Y = torch.empty(M, N, device="cuda", dtype=dt)
    gathered = torch.empty(M, K, device="cuda", dtype=dt)
    flags = torch.zeros(M // 128, dtype=torch.int32, device="cuda")
    maps = torch.empty(32 * 128, dtype=torch.uint8, device="cuda")
    ptrs = (c_void_p * P)(*[s.data_ptr() for s in shards])
    epoch = [0]

    def ag():
        epoch[0] += 1
        rc = lib.lb_gemm_comm_tc(None, W.data_ptr(), Y.data_ptr(), M, N, K, K, K, N, 0, 0,
                                 native.dtype_code(dt), native.dtype_code(dt), 1.0, ptrs, rows, None, 0,
                                 P, 0, maps.data_ptr(), gathered.data_ptr() if a.helpers > 0 else None,
                                 flags.data_ptr(), epoch[0], a.helpers, None, 0, 0, native.stream_ptr())
        native.check(rc, "lb_gemm_comm_tc")

    ms, mn = timer.run(ag)
    out.append(_report("allgather_gemm_staged(1-GPU layout)", [M, N, K], ms, mn, 2.0 * M * N * K,
                       2.0 * (M * K + N * K + M * N)))
    ref = torch.cat(shards).float() @ W.float().t()
    err = float((Y.float() - ref).abs().max() / ref.abs().max())
    # GEMM -> reduce-scatter: K slice of this "rank", rows of the result owned half / half
    A = torch.randn(M, K, device="cuda", dtype=dt)
    B = torch.randn(N, K, device="cuda", dtype=dt)
    own = torch.zeros(rows, N, device="cuda", dtype=torch.float32)
    slot = torch.zeros(rows, N, device="cuda", dtype=torch.float32)
    rs = (c_void_p * P)(own.data_ptr(), slot.data_ptr())

    def rsf():
        rc = lib.lb_gemm_comm_tc(A.data_ptr(), B.data_ptr(), None, M, N, K, K, K, N, 0, 0,
                                 native.dtype_code(dt), native.DT_F32, 1.0, None, 0, None, 0, P, 0, None,
                                 None, None, 0, 0, rs, rows, 1, native.stream_ptr())
        native.check(rc, "lb_gemm_comm_tc")

    ms, mn = timer.run(rsf)
    out.append(_report("gemm_reduce_scatter(1-GPU layout)", [M, N, K], ms, mn, 2.0 * M * N * K,
                       2.0 * (M * K + N * K) + 4.0 * M * N))
    ref2 = A.float() @ B.float().t()
    err2 = float((torch.cat([own, slot]) - ref2).abs().max() / ref2.abs().max())
    print(json.dumps({"max_rel_err_allgather_gemm": err, "max_rel_err_reduce_scatter": err2}))
    return out


def case_linear_wgrad(a, timer):
    """grad[n, k] += dy[m, n]^T x[m, k] for a short mini-batch of m rows (rank-m update)."""
    from lbann_b200.ops import nn
    dt = _dtype(a.dtype)
    dy = torch.randn(a.m, a.n, device="cuda", dtype=dt)
    x = torch.randn(a.m, a.k, device="cuda", dtype=dt)
    grad = torch.zeros(a.n, a.k, device="cuda")
    ms, mn = timer.run(lambda: nn._weight_grad(dy, x, grad))
    return _report("linear_wgrad", [a.m, a.n, a.k], ms, mn, 2.0 * a.m * a.n * a.k,
                   8.0 * a.n * a.k + 2.0 * a.m * (a.n + a.k))


def case_bn(a, timer):
    """Batch normalisation + ReLU over a 2-D activation [batch, cin, size, size]: forward
    (statistics pass + apply pass) and, with ``--bwd``, backward (reduction pass + apply pass)."""
    from lbann_b200.ops import nn
    dt = _dtype(a.dtype)
    N, C, S = a.batch, a.cin, a.size
    x = torch.randn(N, S, S, C, device="cuda", dtype=dt).permute(0, 3, 1, 2).requires_grad_(True)
    sh = nn.WeightHandle(torch.ones(C, device="cuda").requires_grad_(True), torch.zeros(C, device="cuda"))
    bh = nn.WeightHandle(torch.zeros(C, device="cuda").requires_grad_(True), torch.zeros(C, device="cuda"))
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    elems = float(N) * S * S * C

    def fwd():
        return nn.batch_norm(x, sh, bh, rm, rv, True, 1e-5, 0.9, act=native.ACT_RELU)

    ms, mn = timer.run(fwd)
    out = [_report("bn_relu_fwd", [N, C, S], ms, mn, 0.0, 2.0 * elems * 3)]
    if a.bwd:
        y = fwd()
        dy = torch.randn_like(y)
        ms, mn = timer.run(lambda: y.backward(dy, retain_graph=True))
        out.append(_report("bn_relu_bwd", [N, C, S], ms, mn, 0.0, 2.0 * elems * 6))
    return out


def case_optimizer(a, timer):
    from lbann_b200.ops.optim import ParameterArena
    arena = ParameterArena(torch.device("cuda"), _dtype(a.dtype))
    n = a.m * a.k
    slot = arena.reserve("w", (a.m, a.k))
    arena.materialise()
    slot.kind = a.opt
    slot.hp = {"learn_rate": 1e-3, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8, "momentum": 0.9}
    arena.grad.normal_()
    ms, mn = timer.run(lambda: arena.step())
    states = {"sgd": 1, "adam": 2}.get(a.opt, 2)
    return _report(f"optimizer_{a.opt}", [n], ms, mn, 0.0,
                   4.0 * n * (2 + 2 * states + 1) + 2.0 * n)


def case_attention(a, timer):
    """Fused causal attention (csrc/attention_tc.cu) on a packed [batch, seq, 3 * heads * 128]
    projection; with --bwd the backward kernels (delta, key/value side, query side) are timed
    as well, and --sdpa times torch's scaled_dot_product_attention on the same problem."""
    import math
    from lbann_b200.ops import attention as att
    dt = _dtype(a.dtype)
    B, H, S, D = a.batch, a.heads, a.seq, 128
    E = H * D
    qkv = (torch.randn(B, S, 3 * E, device="cuda") * 0.5).to(dt).requires_grad_(True)
    scale = 1.0 / math.sqrt(D)
    causal = not a.no_causal
    flops_fwd = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
    io = 2.0 * B * S * E * 4
    ms, mn = timer.run(lambda: att.attention_packed(qkv, H, scale, causal))
    out = [_report("attention_fwd", [B, H, S, D], ms, mn, flops_fwd, io)]
    if a.bwd:
        y = att.attention_packed(qkv, H, scale, causal)
        g = torch.randn_like(y)
        ms, mn = timer.run(lambda: torch.autograd.grad(y, qkv, g, retain_graph=True))
        # backward runs seven products where forward runs two (P is recomputed on both sides)
        out.append(_report("attention_bwd", [B, H, S, D], ms, mn, 3.5 * flops_fwd, 2.5 * io))
    if a.sdpa:
        import torch.nn.functional as F
        q, k, v = (qkv.detach()[:, :, i * E:(i + 1) * E].reshape(B, S, H, D).transpose(1, 2).contiguous()
                   .requires_grad_(True) for i in range(3))
        ms, mn = timer.run(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=causal))
        out.append(_report("sdpa_fwd", [B, H, S, D], ms, mn, flops_fwd, io))
        if a.bwd:
            y = F.scaled_dot_product_attention(q, k, v, is_causal=causal)
            g = torch.randn_like(y)
            ms, mn = timer.run(lambda: torch.autograd.grad(y, (q, k, v), g, retain_graph=True))
            out.append(_report("sdpa_bwd", [B, H, S, D], ms, mn, 2.5 * flops_fwd, 2.5 * io))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=["gemm", "gemm_comm", "conv", "pool", "optimizer", "linear_wgrad", "bn",
                                     "attention"])
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--no-causal", action="store_true")
    ap.add_argument("--sdpa", action="store_true", help="also time torch's scaled_dot_product_attention")
    ap.add_argument("--dtype", default="bf16", choices=["fp16", "bf16"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--cin", type=int, default=32)
    ap.add_argument("--cout", type=int, default=64)
    ap.add_argument("--size", type=int, default=64)
    ap.add_argument("--ksize", type=int, default=3)
    ap.add_argument("--act", action="store_true")
    ap.add_argument("--pool", default="none", choices=["none", "separate", "fused"])
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--opt", default="adam")
    ap.add_argument("--helpers", type=int, default=6, help="copying CTAs of the staged all-gather")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a GPU")
    timer = _Timer(a.iters, a.warmup, flush=not a.no_flush)
    {"gemm": case_gemm, "gemm_comm": case_gemm_comm, "conv": case_conv, "pool": case_pool,
     "optimizer": case_optimizer, "linear_wgrad": case_linear_wgrad, "bn": case_bn,
     "attention": case_attention}[a.case](
        a, timer)
    native.consume_status()


if __name__ == "__main__":
    main()
