#!/usr/bin/env python
"""Headline benchmark: CosmoFlow 128^3 with spatial (distconv) parallelism, samples/s, plus
the two other workloads of the reference's headline metric as ``extra`` entries.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference ...                      # the unmodified reference
    python bench.py --impl torch ...                          # PyTorch + cuDNN + NCCL arm only

``value`` - CosmoFlow (the reference's distconv benchmark): 4-channel 128^3 volumes, fp16,
log-normal inputs, 4 regression targets uniform in [-1, 1]; five blocks of conv3d 3x3x3
(32, 64, 128, 256, 256 channels) + leaky ReLU + max-pool 2, then fully-connected
2048 -> 256 -> 4, MSE loss, Adam lr 1e-3 (beta 0.9 / 0.99, eps 1e-8); global mini-batch 8 at
every GPU count (strong scaling), depth dimension split over the GPUs with halo width 1.

``extra.resnet50`` - ResNet-50, bf16 compute / fp32 master weights, per-GPU mini-batch 256
(weak scaling), SGD momentum 0.9, weight decay 1e-4, data parallel.
``extra.gpt`` - GPT decoder, 24 layers, d_model 2048, 16 heads, FFN 8192, sequence 2048,
vocabulary 50304, bf16, Adam beta (0.9, 0.95) lr 3e-4, 8 sequences per GPU (64 at 8 GPUs).
Each extra entry carries this framework's numbers and, under ``torch``, the same model
through PyTorch + cuDNN / cuBLAS / SDPA + NCCL (DDP) measured in the same run.

Two numbers per workload.  ``value`` / ``ms_per_step`` are timed on the device: CUDA events
around exactly K steps whose input mini-batches already sit in device memory, max over
ranks; the K-step region is repeated ``--repeats`` times back to back and the MEDIAN region
is reported, so that the clock sampler sees more than a second of load.  ``e2e`` runs the
same steps through the public API (``trainer.train``): every step copies its mini-batch
from pinned host memory to the device and reads the loss back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

BASELINE_SAMPLES_PER_S = 57.0   # reference CI expectation: 8x V100, mb 2, 0.035 s / step
GLOBAL_BATCH = 8
# diagnosis only (how the kernels behave on the per-GPU share of a larger job): any other value
# is reported in `config.global_batch` and is not the headline configuration
GLOBAL_BATCH = int(os.environ.get("LBANN_BENCH_GLOBAL_BATCH", GLOBAL_BATCH))
WIDTH = 128


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    # The reference is a CMake superbuild whose distributed linear algebra, collectives and
    # distconv kernels (Hydrogen, Aluminum, DiHydrogen) are fetched from the network; the one
    # offline pip install of the reference tree answers that the directory is not installable:
    # neither setup.py nor pyproject.toml is found.
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is a CMake superbuild (no setup.py/pyproject.toml; "
                                     "Hydrogen/Aluminum/DiHydrogen must be fetched from the network), "
                                     "so it cannot be installed offline"}))
    return 0


# ------------------------------------------------------------------------ experiments
def cosmoflow_experiment(lbann, n_gpus, pool, depth_groups=0):
    from lbann_b200.models.cosmoflow import construct_cosmoflow_model, synthetic_reader
    depth = depth_groups if depth_groups > 0 else n_gpus      # left-over ranks become sample groups
    ps = lbann.get_parallel_strategy_args(depth_groups=depth) if (n_gpus > 1 and depth > 1) else None
    model = construct_cosmoflow_model(WIDTH, 4, 4, num_epochs=1, channels=(32, 64, 128, 256, 256),
                                      pool_mode="max", parallel_strategy=ps, conv_bias=False)
    model.amp = lbann.AmpOptions(enabled=True, init_scale=128.0)
    trainer = lbann.Trainer(mini_batch_size=GLOBAL_BATCH, random_seed=1)
    reader = synthetic_reader(pool, WIDTH, 4, 4, pool=pool)
    opt = lbann.Adam(learn_rate=1e-3, beta1=0.9, beta2=0.99, eps=1e-8)
    return lbann.proto.serialize.build_experiment(trainer=trainer, model=model, data_reader=reader,
                                                  optimizer=opt)


def resnet50_experiment(lbann, world, batch, image=224):
    from lbann_b200.models import ResNet50, construct_classifier
    model = construct_classifier(ResNet50(1000, bn_statistics_group_size=1), 1000,
                                 l2_weight_decay=1e-4)
    r = lbann.reader_pb2.Reader()
    r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
    r.synth_dimensions = f"3 {image} {image}"
    r.num_samples = 2 * batch * world
    r.num_labels = 1000
    r.synth_pool_size = 2 * batch * world
    dr = lbann.reader_pb2.DataReader()
    dr.reader.append(r)
    return lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=batch * world, random_seed=1), model=model,
        data_reader=dr, optimizer=lbann.SGD(learn_rate=0.1, momentum=0.9))


def gpt_experiment(lbann, world, batch, layers=24, d_model=2048, heads=16, seq=2048, vocab=50304):
    from lbann_b200.models.transformer import construct_gpt_model
    model = construct_gpt_model(vocab_size=vocab, seq_len=seq, d_model=d_model, num_heads=heads,
                                num_layers=layers, ffn_dim=4 * d_model)
    r = lbann.reader_pb2.Reader()
    r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
    r.synth_dimensions = str(seq + 1)
    r.num_samples = 2 * batch * world
    r.synth_distribution = f"randint:{vocab}"
    r.synth_pool_size = 2 * batch * world
    dr = lbann.reader_pb2.DataReader()
    dr.reader.append(r)
    return lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=batch * world, random_seed=1), model=model,
        data_reader=dr, optimizer=lbann.Adam(learn_rate=3e-4, beta1=0.9, beta2=0.95, eps=1e-8))


# ------------------------------------------------------------------------ measurement
def _amp_snapshot(model):
    """(loss scale, consecutive skipped steps, clean steps) read from the device."""
    st = getattr(model, "_amp_state", None)
    if st is None:
        return None
    v = st.tolist()
    return {"scale": v[0], "consecutive_skipped": v[3], "clean_steps": v[2]}


def measure(trainer, model, comm, steps, warm, repeats, samples_per_step, graph, sampler=None,
            field_dtypes=None):
    """Device-timed and end-to-end numbers of one built model (see the module docstring)."""
    import torch
    from lbann_b200.callbacks import ExecCallback
    from lbann_b200.ops import native
    dc = trainer.data_coordinator
    if field_dtypes:
        dc.field_dtypes = field_dtypes
    dc.cache_collated = True
    dev = trainer.device
    dc.start_epoch("training")
    resident = []
    for _ in range(2):
        b = dc.next_batch("training")
        resident.append(({k: v.clone() for k, v in b.tensors.items()}, b.global_size))
    torch.cuda.synchronize()
    # The synthetic task has no signal (random volumes, random targets), so a long run at the
    # prescribed learning rate is a random walk of the weights that ends in fp16 overflow after a
    # few hundred steps.  Every timed region therefore starts from the same initial state: the
    # snapshot is written back (untimed), `warm` untimed steps follow, then the K timed steps.
    initial = model.snapshot_state()
    first_loss = None
    for i in range((4 if graph else 0) + warm):     # ordinary steps, the capture, warm-up: untimed
        t, g = resident[i % 2]
        model.train_step(t, g)
        if first_loss is None:
            first_loss = float(model.last_objective)
    torch.cuda.synchronize()
    status = native.consume_status(False)
    comm.barrier("world")
    if sampler is not None:
        sampler.start()
    # AMP: a skipped step does less work (no update).  The schedule's counters live on the
    # device; a timed region is clean when the clean-step counter grew by exactly K.
    region_ms, skipped = [], 0
    launches = 0
    for _ in range(repeats):
        model.restore_state(initial)
        for i in range(warm):
            t, g = resident[i % 2]
            model.train_step(t, g)
        amp0 = _amp_snapshot(model)
        launches0 = native.launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        comm.barrier("world")
        torch.cuda.synchronize()
        e0.record()
        for i in range(steps):
            t, g = resident[i % 2]      # two resident mini-batches alternate
            model.train_step(t, g)
        e1.record()
        torch.cuda.synchronize()
        comm.barrier("world")
        launches = native.launches() - launches0
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        comm.allreduce(ms, "world", "max")
        region_ms.append(float(ms.item()))
        if amp0 is not None:
            now = _amp_snapshot(model)
            grew = (now["clean_steps"] - amp0["clean_steps"]) % max(model.amp_interval, 1)
            if now["consecutive_skipped"] > 0 or (grew != steps % max(model.amp_interval, 1)):
                skipped += 1
    last_loss = float(model.last_objective)
    region_ms.sort()
    ms = region_ms[len(region_ms) // 2]

    # ---- end to end through the public API
    losses = []

    class ReadLoss(ExecCallback):
        """Reads the objective of EVERY step on the host.  The copy into pinned memory is
        enqueued behind the step and its value is taken one step later, so the host does not
        stall the device once per step (a blocking read cost 0.1 ms per step on one GPU and
        0.4-0.65 ms on 2-4, where every rank's stall also delays its neighbours' halos)."""

        def __init__(self):
            self.pinned = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(2)]
            self.events = [None, None]
            self.k = 0

        def _take(self, j):
            if self.events[j] is not None:
                self.events[j].synchronize()
                losses.append(float(self.pinned[j][0]))
                self.events[j] = None

        def on_batch_end(self, m):
            i = self.k & 1
            self._take(i ^ 1)                               # the previous step's value
            self.pinned[i].copy_(m.last_objective.detach().reshape(1).float(), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev
            self.k += 1

        def flush(self):
            self._take((self.k & 1) ^ 1)
            self._take(self.k & 1)

    reader = ReadLoss()
    model.callbacks.append(reader)
    model.restore_state(initial)
    dc.start_epoch("training")
    trainer.context(model, "training").step = 0
    trainer.train(model, num_batches=warm)               # untimed warm-up of the whole pipeline
    reader.flush()
    torch.cuda.synchronize()
    comm.barrier("world")
    h2d0, n0 = dc.total_h2d_bytes, len(losses)
    # like the device-timed number: the median of a few regions of K steps each
    e2e_regions = []
    n_regions = max(1, min(repeats, 3))
    for _ in range(n_regions):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        comm.barrier("world")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record()
        trainer.context(model, "training").step = 0
        trainer.train(model, num_batches=steps)
        reader.flush()                                   # the last step's value, inside the timed region
        e1.record()
        torch.cuda.synchronize()
        comm.barrier("world")
        region = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
        tmax = torch.tensor([region], device=dev)
        comm.allreduce(tmax, "world", "max")
        e2e_regions.append(float(tmax.item()))
    e2e_regions.sort()
    e2e_ms = e2e_regions[len(e2e_regions) // 2]
    h2d = (dc.total_h2d_bytes - h2d0) / max(steps * n_regions, 1)
    status |= native.consume_status(False)
    return {"ms_per_step": ms / steps, "region_ms": region_ms, "e2e_ms_per_step": e2e_ms / steps,
            "e2e_steps": len(losses) - n0, "e2e_region_ms": [round(v, 3) for v in e2e_regions], "h2d_bytes_per_step": int(h2d), "gpu_launches": int(launches),
            "first_loss": first_loss, "final_loss": last_loss, "device_status": int(status),
            "amp": _amp_snapshot(model), "regions_with_skipped_steps": skipped,
            "cuda_graph": bool(getattr(model, "_graph_mode", False)),
            "samples_per_s": samples_per_step / (ms / steps) * 1e3,
            "e2e_samples_per_s": samples_per_step / (e2e_ms / steps) * 1e3}


def _release(trainer):
    import gc
    import torch
    trainer.shutdown()
    gc.collect()
    torch.cuda.empty_cache()


def run_extra(name, args, world, rank, comm_holder):
    """ResNet-50 / GPT through this framework; returns a dict for the JSON line."""
    import torch
    import lbann_b200 as lbann
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.utils import options as opts
    o = opts.reset()
    o.set("default_dtype", "bf16")
    if not args.no_graph:
        o.set("use_cuda_graph", True)
    if name == "resnet50":
        batch = args.resnet_batch
        exp = resnet50_experiment(lbann, world, batch)
        per_step, unit = batch * world, "images/s"
        cfg = {"model": "ResNet-50, 3x224x224, 1000 classes", "global_batch": batch * world,
               "per_gpu_batch": batch, "optimizer": "SGD momentum 0.9, weight decay 1e-4",
               "parallelism": f"dp{world}", "scaling": "weak"}
        steps = max(min(args.steps, 10), 3)
    else:
        batch = args.gpt_batch
        exp = gpt_experiment(lbann, world, batch, layers=args.gpt_layers)
        per_step, unit = batch * world * 2048, "tokens/s"
        cfg = {"model": f"GPT {args.gpt_layers} layers, d_model 2048, 16 heads, FFN 8192, seq 2048, "
                        "vocab 50304, pre-LN, GELU, learned positions",
               "global_batch": batch * world, "seq_len": 2048,
               "optimizer": "Adam lr 3e-4 beta (0.9, 0.95)",
               "parallelism": f"dp{world}, optimizer state and update sharded over the ranks",
               "scaling": "weak"}
        steps = max(min(args.steps, 5), 2)
    trainer = ExecTrainer(exp)
    model = trainer.build_model(exp.model)
    m = measure(trainer, model, trainer.comm, steps, 3, max(args.repeats // 3, 1), per_step,
                not args.no_graph)
    out = {"impl": "lbann_b200", "unit": unit, "value": round(m["samples_per_s"], 2),
           "ms_per_step": round(m["ms_per_step"], 3), "steps": steps, "dtype": "bf16",
           "e2e": {"value": round(m["e2e_samples_per_s"], 2), "unit": unit,
                   "ms_per_step": round(m["e2e_ms_per_step"], 3),
                   "h2d_bytes_per_step": m["h2d_bytes_per_step"], "d2h_bytes_per_step": 4},
           "gpu_launches": m["gpu_launches"], "first_loss": m["first_loss"], "final_loss": m["final_loss"],
           "device_status": m["device_status"], "cuda_graph": m["cuda_graph"], "config": cfg}
    _release(trainer)
    return out


def ours(args):
    import torch
    import lbann_b200 as lbann
    from lbann_b200.exec.trainer import ExecTrainer
    from lbann_b200.utils import options as opts

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            # convenience: re-launch under torchrun
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
                   str(29400 + os.getpid() % 500), os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")

    o = opts.reset()
    o.set("default_dtype", "fp16")
    if not args.no_graph:
        o.set("use_cuda_graph", True)       # the step is captured once and replayed
    steps, warm = args.steps, max(args.warmup, 3)
    pool = 2 * GLOBAL_BATCH
    # the synthetic data set is two mini-batches long; epochs simply repeat, so the collated
    # pinned host batches are built once and every step pays only for its own transfers
    exp = cosmoflow_experiment(lbann, world, pool, args.depth_groups)
    trainer = ExecTrainer(exp)
    model = trainer.build_model(exp.model)
    comm = trainer.comm
    sampler = ClockSampler(local_rank) if rank == 0 else None
    m = measure(trainer, model, comm, steps, warm, args.repeats, GLOBAL_BATCH, not args.no_graph,
                sampler, {"samples": torch.float16, "responses": torch.float16})
    clocks = sampler.stop() if sampler is not None else None
    phase = model._phase_timer.report() if getattr(model, "_phase_timer", None) is not None else None
    halo = None
    if trainer.distconv is not None:
        halo = {"tensors_with_halo_planes": len(trainer.distconv._halo_tensors),
                "interior_copies": trainer.distconv.interior_copies}
    sharded = model.arena.shard is not None
    value = m["samples_per_s"]
    out = {
        "metric": "CosmoFlow distconv training throughput", "value": round(value, 3),
        "unit": "samples/s", "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": round(m["ms_per_step"], 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(value / BASELINE_SAMPLES_PER_S, 3), "dtype": "fp16",
        "data": "synthetic", "impl": "lbann_b200",
        "config": {"model": "CosmoFlow 128^3, conv3d 3x3x3 (32,64,128,256,256)+leakyReLU+maxpool2, "
                            "FC 2048-256-4, MSE, random init",
                   "optimizer": "Adam lr 1e-3 beta1 0.9 beta2 0.99 eps 1e-8, AMP initial loss scale 128",
                   "global_batch": GLOBAL_BATCH, "seq_len": None,
                   "parallelism": (f"distconv depth x{args.depth_groups or world}"
                                   + (f" x {world // args.depth_groups} sample groups"
                                      if args.depth_groups and args.depth_groups < world else "")
                                   + ", halo exchange inside the convolution kernels, optimizer "
                                     "sharded over the ranks") if world > 1 else "single GPU",
                   "timing": f"CUDA events, max over ranks, median of {args.repeats} regions of {steps} "
                             "steps; two resident 134 MB fp16 mini-batches alternate so inputs exceed "
                             "the 126 MB L2",
                   "cuda_graph": m["cuda_graph"]},
        "e2e": {"value": round(m["e2e_samples_per_s"], 3), "unit": "samples/s",
                "ms_per_step": round(m["e2e_ms_per_step"], 4), "region_ms": m["e2e_region_ms"],
                "h2d_bytes_per_step": m["h2d_bytes_per_step"], "d2h_bytes_per_step": 4,
                "path": "lbann_b200 ExecTrainer.train: pinned host mini-batch -> device every step; the "
                        "loss of every step is copied to pinned host memory behind the step and read "
                        "one step later"},
        "gpu_launches": m["gpu_launches"], "first_loss": m["first_loss"], "final_loss": m["final_loss"],
        "amp": m["amp"], "regions_with_skipped_steps": m["regions_with_skipped_steps"],
        "region_ms": [round(v, 3) for v in m["region_ms"]],
        "device_status": m["device_status"], "clocks": clocks,
        "distconv": halo, "sharded_optimizer": sharded,
        "optimizer_state_bytes_per_rank": int(model.arena.state_bytes()),
        "cpu_cores_bound": len(getattr(trainer, "cpu_binding", None) or ()) or None,
    }
    if phase is not None and rank == 0:
        # LBANN_PHASE_TIMING=1: (device ms, host ms) per phase of the step, on stderr
        print("phase timing:", phase, file=sys.stderr)
    _release(trainer)

    # ------------------------------------------------------------ the other two workloads
    extra = {}
    wanted = [w for w in args.workloads.split(",") if w in ("resnet50", "gpt")]
    for name in wanted:
        entry = {}
        try:
            entry.update(run_extra(name, args, world, rank, comm))
        except Exception as e:      # an extra workload never takes the headline line down
            entry["error"] = f"{type(e).__name__}: {e}"[:400]
            torch.cuda.synchronize()
        if not args.no_torch_arm:
            try:
                entry["torch"] = torch_extra(name, args, world, rank, local_rank)
            except Exception as e:
                entry["torch"] = {"error": f"{type(e).__name__}: {e}"[:400]}
        extra[name] = entry
    if not args.no_torch_arm:
        try:
            from baseline.torch_cosmoflow import measure_torch
            out["torch_arm"] = measure_torch(steps, warm, GLOBAL_BATCH, WIDTH)
        except Exception as e:
            out["torch_arm"] = {"error": f"{type(e).__name__}: {e}"[:400]}
    if extra:
        out["extra"] = extra
    rc = 0
    if m["regions_with_skipped_steps"]:
        out["invalid"] = "automatic mixed precision skipped steps inside a timed region"
        rc = 3
    if rank == 0:
        print(json.dumps(out))
    comm.finalize()
    return rc


def torch_extra(name, args, world, rank, local_rank):
    from baseline.torch_models import measure_torch_model
    return measure_torch_model(name, args, world, rank, local_rank)


def torch_arm(args):
    from baseline.torch_cosmoflow import run
    return run(args, GLOBAL_BATCH, WIDTH, BASELINE_SAMPLES_PER_S, ClockSampler)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=10, help="timed regions of --steps steps; the median counts")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host")
    ap.add_argument("--workloads", default=os.environ.get("LBANN_BENCH_WORKLOADS", "cosmoflow,resnet50,gpt"),
                    help="comma list; cosmoflow is always the headline value")
    ap.add_argument("--no-torch-arm", action="store_true", help="skip the PyTorch comparison arms")
    ap.add_argument("--depth-groups", type=int, default=int(os.environ.get("LBANN_BENCH_DEPTH_GROUPS", "0")),
                    help="CosmoFlow: ranks per depth partition (default: all GPUs); the other ranks "
                         "multiply the sample groups")
    ap.add_argument("--resnet-batch", type=int, default=256, help="per-GPU mini-batch of the ResNet-50 entry")
    ap.add_argument("--gpt-batch", type=int, default=8, help="sequences per GPU of the GPT entry")
    ap.add_argument("--gpt-layers", type=int, default=24)
    a = ap.parse_args()
    if a.impl == "reference":
        sys.exit(reference_arm(a))
    if a.impl == "torch":
        sys.exit(torch_arm(a))
    sys.exit(ours(a))
