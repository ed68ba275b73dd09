"""Reporting, learning-rate schedules, gradient handling and verification callbacks.

Each class names the reference source it mirrors.  Output lines parsed by the reference's
CI (objective / metric / timing reports) keep their exact wording.
"""
from __future__ import annotations

import math
import statistics
import sys
import time

import torch

from .base import (ExecCallback, is_master, is_trainer_master, mode_string, register,
                   select_layers, select_weights)


def _trainer_rank(model):
    return model.comm.trainer_rank if model.comm is not None else 0


# =============================================================================== reporting
@register("print")
class PrintStatistics(ExecCallback):
    """src/callbacks/print_statistics.cpp:88-115,178-267"""

    def __init__(self, params=None):
        super().__init__(params)
        self.interval = int(getattr(params, "interval", 0) or 1)
        self.global_only = bool(getattr(params, "print_global_stat_only", False))

    def on_epoch_begin(self, model):
        ctx = model.ctx
        if ctx.epoch % self.interval == 0 and is_master(model):
            dc = model.trainer.data_coordinator
            line = "-" * 92
            it = [dc.iterations_per_epoch(m) for m in ("training", "validation", "testing", "tournament")]
            mb = [dc.mini_batch_size(m) for m in ("training", "validation", "testing", "tournament")]
            last = [dc.last_mini_batch_size(m) for m in ("training", "validation", "testing", "tournament")]
            print(line)
            print(f"[{ctx.epoch}] Epoch : stats formated [tr/v/te/to] iter/epoch = "
                  f"[{it[0]}/{it[1]}/{it[2]}/{it[3]}]")
            print(f"{'  Global MB =':>23} [{mb[0]:4d}/{mb[1]:4d}/{mb[2]:4d}/{mb[3]:4d}]"
                  f"  Global last MB = [{last[0]:4d}/{last[1]:4d}/{last[2]:4d}/{last[3]:4d}]")
            print(line, flush=True)

    def _report(self, model, mode):
        obj, mets, samples = model.reduce_statistics(mode)
        comm = model.comm
        ms = mode_string(model, mode)
        ntr = comm.num_trainers if comm is not None else 1
        if ntr > 1:
            rows = comm.intertrainer_gather_object((obj, mets, samples))
            if not is_master(model):
                return
            if not self.global_only:
                for i, (o, mm, _) in enumerate(rows):
                    print(f"{model.name} (instance {i}) {ms} objective function : {o:.6g}")
            tot = sum(r[2] for r in rows) or 1
            print(f"{model.name} global average {ms} objective function : "
                  f"{sum(r[0] * r[2] for r in rows) / tot:.6g}")
            for k, met in enumerate(model.metrics):
                scores = [r[1][k] for r in rows]
                if not self.global_only:
                    for i, s in enumerate(scores):
                        print(f"{model.name} (instance {i}) {ms} {met.name} : {s:.6g}{met.unit}")
                avg = sum(s * r[2] for s, r in zip(scores, rows)) / tot
                sd = statistics.stdev(scores) if len(scores) > 1 else 0.0
                for tag, v in (("global average", avg), ("global min", min(scores)),
                               ("global max", max(scores)), ("global stdev", sd)):
                    print(f"{model.name} ({tag}) {ms} {met.name} : {v:.6g}{met.unit}")
            sys.stdout.flush()
            return
        if is_trainer_master(model):
            r = _trainer_rank(model)
            out = [f"{model.name} (instance {r}) {ms} objective function : {obj:.6g}"]
            for met, v in zip(model.metrics, mets):
                out.append(f"{model.name} (instance {r}) {ms} {met.name} : {v:.6g}{met.unit}")
            print("\n".join(out), flush=True)

    def on_epoch_end(self, model):
        if model.ctx.epoch % self.interval == 0:
            self._report(model, "training")

    def on_validation_end(self, model):
        self._report(model, "validation")

    def on_test_end(self, model):
        self._report(model, "testing")


@register("timer")
class Timer(ExecCallback):
    """src/callbacks/timer.cpp:216-283"""

    def __init__(self, params=None):
        super().__init__(params)
        self.skip = int(getattr(params, "skip_steps", 0) or 0)
        self.start = {}
        self.batch_start = {}
        self.times = {}

    def _begin(self, model, mode):
        self.start[mode] = time.perf_counter()
        self.times[mode] = []

    def _batch_begin(self, model, mode):
        self.batch_start[mode] = time.perf_counter()

    def _batch_end(self, model, mode):
        if model.device.type == "cuda" and getattr(model.trainer, "timer_sync", False):
            torch.cuda.synchronize()
        self.times.setdefault(mode, []).append(time.perf_counter() - self.batch_start.get(mode, time.perf_counter()))

    def _end(self, model, mode):
        if model.device.type == "cuda":
            torch.cuda.synchronize()
        run = time.perf_counter() - self.start.get(mode, time.perf_counter())
        t = self.times.get(mode, [])[self.skip:] if mode == "training" else self.times.get(mode, [])
        if not is_trainer_master(model):
            return
        r = _trainer_rank(model)
        ms = mode_string(model, mode)

        def f(v):
            return "N/A" if (v is None or math.isnan(v)) else f"{v:.6g}s"
        mean = statistics.fmean(t) if t else float("nan")
        med = statistics.median(t) if t else float("nan")
        sd = statistics.stdev(t) if len(t) > 1 else float("nan")
        print(f"{model.name} (instance {r}) {ms} run time : {run:.6g}s")
        print(f"{model.name} (instance {r}) {ms} mini-batch time statistics : {f(mean)} mean, "
              f"{f(med)} median, {f(max(t) if t else None)} max, {f(min(t) if t else None)} min, "
              f"{f(sd)} stdev", flush=True)
        model.trainer.last_timing[mode] = {"run": run, "mean": mean, "median": med}

    def on_epoch_begin(self, model): self._begin(model, "training")
    def on_epoch_end(self, model): self._end(model, "training")
    def on_batch_begin(self, model): self._batch_begin(model, "training")
    def on_batch_end(self, model): self._batch_end(model, "training")
    def on_validation_begin(self, model): self._begin(model, "validation")
    def on_validation_end(self, model): self._end(model, "validation")
    def on_test_begin(self, model): self._begin(model, "testing")
    def on_test_end(self, model): self._end(model, "testing")
    def on_batch_evaluate_begin(self, model, mode): self._batch_begin(model, mode)
    def on_batch_evaluate_end(self, model, mode): self._batch_end(model, mode)


@register("progress_bar")
class ProgressBar(ExecCallback):
    """src/callbacks/progress_bar.cpp"""

    def __init__(self, params=None):
        super().__init__(params)
        p = params
        self.interval = int(getattr(p, "interval", 0) or 1)
        self.newline = int(getattr(p, "newline_interval", 0) or 0)
        self.avg_len = int(getattr(p, "moving_average_length", 0) or 10)
        self.width = int(getattr(p, "bar_width", 0) or 30)
        self.sci = bool(getattr(p, "scientific_notation", False))
        self.mem = bool(getattr(p, "print_mem_usage", False))
        self.hist, self.t0 = [], None

    def on_epoch_begin(self, model):
        self.hist, self.t0 = [], time.perf_counter()

    def on_batch_end(self, model):
        if not is_master(model):
            return
        now = time.perf_counter()
        self.hist = (self.hist + [now])[-self.avg_len - 1:]
        step = model.ctx.step_in_epoch
        total = max(model.trainer.data_coordinator.iterations_per_epoch("training"), 1)
        if step % self.interval and step != total:
            return
        rate = (len(self.hist) - 1) / max(self.hist[-1] - self.hist[0], 1e-9) if len(self.hist) > 1 else 0.0
        fill = int(self.width * step / total)
        loss = float(model.last_objective) if model.last_objective is not None else float("nan")
        ls = f"{loss:.3e}" if self.sci else f"{loss:.4f}"
        extra = ""
        if self.mem and model.device.type == "cuda":
            extra = f" mem {torch.cuda.memory_allocated() / 2**30:.2f} GiB"
        end = "\n" if (self.newline and step % self.newline == 0) or step == total else "\r"
        print(f"Epoch {model.ctx.epoch} [{'#' * fill}{'.' * (self.width - fill)}] {step}/{total} "
              f"{rate:.2f} it/s loss {ls}{extra}", end=end, flush=True)


@register("print_model_description")
class PrintModelDescription(ExecCallback):
    """src/callbacks/print_model_description.cpp"""

    def on_setup_end(self, model):
        if is_master(model):
            print(model.describe(), flush=True)


@register("compute_model_size")
class ComputeModelSize(ExecCallback):
    """Number of parameters written into a constant weights object
    (src/callbacks/compute_model_size.cpp)."""

    def on_batch_end(self, model):
        if model.ctx.step % self.batch_interval:
            return
        n = sum(w.slot.count for w in model.weights if w.has_optimizer())
        out = model.weights_by_name.get(self.params.output_name)
        if out is not None:
            out.set_values(torch.full(out.shape, float(n)))
        elif is_master(model) and model.ctx.step == 0:
            print(f"{model.name}: model size {n} parameters")


@register("gpu_memory_usage")
class GpuMemoryUsage(ExecCallback):
    """src/callbacks/gpu_memory_usage.cpp"""

    def on_epoch_begin(self, model):
        if model.device.type != "cuda":
            return
        free, total = torch.cuda.mem_get_info()
        used = total - free
        vals = [used / 2**30]
        if model.comm is not None:
            vals = model.comm.trainer_gather_object(used / 2**30)
        if is_trainer_master(model):
            print(f"GPU memory usage statistics : {statistics.fmean(vals):.3f} GiB mean, "
                  f"{statistics.median(vals):.3f} GiB median, {max(vals):.3f} GiB max, "
                  f"{min(vals):.3f} GiB min ({total / 2**30:.1f} GiB total)", flush=True)


@register("memory_profiler")
class MemoryProfiler(ExecCallback):
    """Per-layer activation / weights / optimizer-state accounting with peak tracking
    (src/callbacks/memory_profiler.cpp)."""

    def __init__(self, params=None):
        super().__init__(params)
        self.detailed = bool(getattr(params, "detailed_first_step", False))
        self.layer_bytes = {}
        self.first = True

    def on_setup_end(self, model):
        if not is_master(model):
            return
        wbytes = sum(w.slot.count * 4 for w in model.weights)
        states = sum(w.slot.count * 4 * (2 if w.slot.kind == "adam" else 1)
                     for w in model.weights if w.has_optimizer())
        print(f"MEM: weights {wbytes / 2**20:.2f} MiB, optimizer state {states / 2**20:.2f} MiB, "
              f"gradients {wbytes / 2**20:.2f} MiB")

    def on_layer_forward_begin(self, model, layer, mode):
        if self.first and self.detailed and model.device.type == "cuda":
            torch.cuda.synchronize()
            self._before = torch.cuda.memory_allocated()

    def on_layer_forward_end(self, model, layer, mode):
        if self.first and self.detailed and model.device.type == "cuda":
            torch.cuda.synchronize()
            self.layer_bytes[layer.name] = torch.cuda.memory_allocated() - self._before

    def on_batch_end(self, model):
        if not self.first:
            return
        self.first = False
        if is_master(model):
            if model.device.type == "cuda":
                print(f"MEM: peak allocated after first step {torch.cuda.max_memory_allocated() / 2**20:.2f} MiB")
            for k, v in self.layer_bytes.items():
                print(f"MEM:   layer {k}: {v / 2**20:.3f} MiB of new activations")

    def on_epoch_end(self, model):
        if is_master(model) and model.device.type == "cuda":
            print(f"MEM: epoch {model.ctx.epoch} peak {torch.cuda.max_memory_allocated() / 2**20:.2f} MiB",
                  flush=True)


@register("profiler")
class Profiler(ExecCallback):
    """NVTX ranges around epochs, layers and the optimizer step
    (src/callbacks/profiler.cpp:60-299, include/lbann/utils/profiling.hpp:77-110)."""

    def __init__(self, params=None):
        super().__init__(params)
        self.sync = bool(getattr(params, "sync", False))
        self.skip_init = bool(getattr(params, "skip_init", False))
        self.active = not self.skip_init

    def _push(self, model, name):
        if self.active and model.device.type == "cuda":
            if self.sync:
                torch.cuda.synchronize()
            torch.cuda.nvtx.range_push(name)

    def _pop(self, model):
        if self.active and model.device.type == "cuda":
            if self.sync:
                torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()

    def on_epoch_begin(self, model):
        if self.skip_init and model.ctx.epoch == 1:
            self.active = True
        self._push(model, f"epoch {model.ctx.epoch}")

    def on_epoch_end(self, model): self._pop(model)
    def on_layer_forward_begin(self, model, layer, mode): self._push(model, f"fw {layer.name}")
    def on_layer_forward_end(self, model, layer, mode): self._pop(model)
    def on_backward_prop_begin(self, model): self._push(model, "backward")
    def on_backward_prop_end(self, model): self._pop(model)
    def on_optimize_begin(self, model): self._push(model, "optimize")
    def on_optimize_end(self, model): self._pop(model)


@register("timeline")
class Timeline(ExecCallback):
    """Per-layer start/stop times written per rank (src/callbacks/timeline.cpp)."""

    def __init__(self, params=None):
        super().__init__(params)
        self.dir = getattr(params, "directory", "") or "."
        self.rows, self.t0 = [], {}

    def on_train_begin(self, model):
        self.origin = time.perf_counter()

    def on_layer_forward_begin(self, model, layer, mode):
        if model.device.type == "cuda":
            torch.cuda.synchronize()
        self.t0[layer.name] = time.perf_counter()

    def on_layer_forward_end(self, model, layer, mode):
        if model.device.type == "cuda":
            torch.cuda.synchronize()
        self.rows.append((layer.name, "fp", self.t0[layer.name] - self.origin,
                          time.perf_counter() - self.origin))

    def on_train_end(self, model):
        import os
        os.makedirs(self.dir, exist_ok=True)
        rank = model.comm.rank_in_world if model.comm is not None else 0
        with open(os.path.join(self.dir, f"timeline.m{model.name}.r{rank}.txt"), "w") as f:
            for name, kind, a, b in self.rows:
                f.write(f"{kind}:{name}:{a:.9f}:{b:.9f}\n")


@register("sync_layers")
class SyncLayers(ExecCallback):
    """Synchronise the device (and ranks) after every layer to localise asynchronous
    errors (src/callbacks/sync_layers.cpp)."""

    def on_layer_forward_end(self, model, layer, mode):
        p = self.params
        if p is not None and p.only_input and layer.type != "input":
            return
        if (p is None or p.sync_gpus) and model.device.type == "cuda":
            torch.cuda.synchronize()
            from ..ops import native
            native.consume_status()
        if p is not None and p.sync_mpi and model.comm is not None:
            model.comm.trainer_barrier()


@register("debug")
class Debug(ExecCallback):
    """Prints every hook as it happens (src/callbacks/debug.cpp)."""

    def _say(self, model, what):
        rank = model.comm.rank_in_world if model.comm is not None else 0
        print(f"rank {rank}: {what} (epoch {model.ctx.epoch}, step {model.ctx.step})", flush=True)

    def on_batch_begin(self, model): self._say(model, "starting batch")
    def on_batch_end(self, model): self._say(model, "ending batch")
    def on_layer_forward_begin(self, model, layer, mode): self._say(model, f"{layer.name} forward begin [{mode}]")
    def on_layer_forward_end(self, model, layer, mode): self._say(model, f"{layer.name} forward end [{mode}]")
    def on_backward_prop_begin(self, model): self._say(model, "backward begin")
    def on_backward_prop_end(self, model): self._say(model, "backward end")
    def on_optimize_begin(self, model): self._say(model, "optimize begin")
    def on_optimize_end(self, model): self._say(model, "optimize end")


@register("debug_io")
class DebugIO(ExecCallback):
    """Prints which samples each rank consumed (src/callbacks/debug_io.cpp)."""

    def on_batch_begin(self, model):
        idx = model.trainer.data_coordinator.last_indices("training")
        rank = model.comm.rank_in_world if model.comm is not None else 0
        print(f"rank {rank}: step {model.ctx.step} training samples {list(idx[:8])}"
              f"{'...' if len(idx) > 8 else ''}", flush=True)


@register("disp_io_stats")
class DispIOStats(ExecCallback):
    """src/callbacks/monitor_io.cpp"""

    def on_epoch_end(self, model):
        dc = model.trainer.data_coordinator
        if is_master(model):
            print(f"I/O: {dc.samples_fetched('training')} training samples fetched, "
                  f"{dc.bytes_fetched('training') / 2**20:.1f} MiB, fetch time "
                  f"{dc.fetch_seconds('training'):.3f}s", flush=True)


@register("hang")
class Hang(ExecCallback):
    """Debugging aid: a chosen rank (or all, rank < 0) waits for a debugger on the host
    (src/callbacks/hang.cpp:63-72).  The wait is bounded by LBANN_HANG_SECONDS (default 30)."""

    def setup(self, model):
        import os
        rank = model.comm.rank_in_world if model.comm is not None else 0
        target = int(getattr(self.params, "rank", -1))
        if target < 0 or target == rank:
            limit = float(os.environ.get("LBANN_HANG_SECONDS", "30"))
            print(f"rank {rank} (pid {os.getpid()}) waiting up to {limit}s for a debugger", flush=True)
            t0 = time.time()
            while time.time() - t0 < limit and not os.path.exists(f"/tmp/lbann_release_{os.getpid()}"):
                time.sleep(0.25)


# =============================================================================== learning rate
class _LRSchedule(ExecCallback):
    """Base of the schedules in src/callbacks/learning_rate.cpp: a global schedule is applied
    at the end of every epoch to the selected weights (:87-106)."""

    def setup(self, model):
        self.weights = select_weights(model, getattr(self.params, "weights", ""))
        self.base = {w.name: w.learning_rate for w in self.weights}

    def global_schedule(self, model) -> float:
        return 1.0

    def on_epoch_end(self, model):
        s = self.global_schedule(model)
        if s != 1.0:
            for w in self.weights:
                w.learning_rate = w.learning_rate * s


@register("step_learning_rate")
class StepLearningRate(_LRSchedule):
    """x amt every ``step`` epochs (:135-143)."""

    def global_schedule(self, model):
        step = int(self.params.step) or 1
        return float(self.params.amt) if (model.ctx.epoch + 1) % step == 0 else 1.0


@register("set_learning_rate")
class SetLearningRate(_LRSchedule):
    """Set the rate to ``val`` at epoch ``step`` (:164-172)."""

    def on_epoch_end(self, model):
        if model.ctx.epoch + 1 == int(self.params.step):
            for w in self.weights:
                w.learning_rate = float(self.params.val)


@register("adaptive_learning_rate")
class AdaptiveLearningRate(_LRSchedule):
    """x amt after ``patience`` epochs without objective improvement (:194-227)."""

    def setup(self, model):
        super().setup(model)
        self.best, self.wait = float("inf"), 0

    def global_schedule(self, model):
        mode = "validation" if model.stats["validation"].samples else "training"
        obj, _, _ = model.reduce_statistics(mode)
        if obj < self.best:
            self.best, self.wait = obj, 0
            return 1.0
        self.wait += 1
        if self.wait >= (int(self.params.patience) or 1):
            self.wait = 0
            return float(self.params.amt)
        return 1.0


@register("drop_fixed_learning_rate")
class DropFixedLearningRate(_LRSchedule):
    """x amt at the listed epochs (:268-282)."""

    def global_schedule(self, model):
        return float(self.params.amt) if (model.ctx.epoch + 1) in set(self.params.drop_epoch) else 1.0


@register("linear_growth_learning_rate")
class LinearGrowthLearningRate(_LRSchedule):
    """Linear ramp from the base rate to ``target`` over ``num_epochs`` after ``delay`` (:325-337)."""

    def on_epoch_end(self, model):
        e = model.ctx.epoch + 1
        n, delay = int(self.params.num_epochs) or 1, int(self.params.delay)
        if e < delay or e > delay + n:
            return
        for w in self.weights:
            b = self.base[w.name]
            w.learning_rate = b + (float(self.params.target) - b) * (e - delay) / n


@register("poly_learning_rate")
class PolyLearningRate(_LRSchedule):
    """(start-end) * ((max_iter - iter)/max_iter)^p + end, evaluated every step (:398-419)."""

    def setup(self, model):
        super().setup(model)
        self.max_iter = int(self.params.max_iter)

    def on_train_begin(self, model):
        if not self.max_iter:
            per = model.trainer.data_coordinator.iterations_per_epoch("training")
            self.max_iter = per * (int(self.params.num_epochs) or model.num_epochs)

    def on_epoch_end(self, model):
        pass

    def on_batch_end(self, model):
        it = min(model.ctx.step, self.max_iter)
        frac = ((self.max_iter - it) / max(self.max_iter, 1)) ** (float(self.params.power) or 1.0)
        end = float(self.params.end_lr)
        for w in self.weights:
            w.learning_rate = (self.base[w.name] - end) * frac + end


@register("cosine_decay_learning_rate")
class CosineDecayLearningRate(_LRSchedule):
    """Linear warm-up from ``initial_warmup_learning_rate`` for ``warmup_steps`` steps, then
    lr_min + (lr_max-lr_min) * 0.5 (1 + cos(pi t / decay_steps)), floored at lr_min (:495-515)."""

    def on_epoch_end(self, model):
        pass

    def _lr(self, step):
        p = self.params
        warm = int(p.warmup_steps)
        if step < warm:
            w0 = float(p.initial_warmup_learning_rate)
            return w0 + (float(p.lr_max) - w0) * step / max(warm, 1)
        t = step - warm
        if t >= int(p.decay_steps):
            return float(p.lr_min)
        return float(p.lr_min) + (float(p.lr_max) - float(p.lr_min)) * 0.5 * (
            1.0 + math.cos(math.pi * t / max(int(p.decay_steps), 1)))

    def on_train_begin(self, model):
        for w in self.weights:
            w.learning_rate = self._lr(model.ctx.step)

    def on_batch_end(self, model):
        lr = self._lr(model.ctx.step)
        for w in self.weights:
            w.learning_rate = lr


@register("optimizerwise_adaptive_learning_rate")
class OptimizerwiseAdaptiveLearningRate(_LRSchedule):
    """LARS-style per-weights rate: scale * ||w|| / ||g|| (:108-123, per-optimizer schedule)."""

    def on_epoch_end(self, model):
        pass

    def on_backward_prop_end(self, model):
        scale = float(self.params.scale) or 1.0
        for w in self.weights:
            if w.gradient is None:
                continue
            wn = float(w.values.detach().float().norm())
            gn = float(w.gradient.float().norm())
            if wn > 0 and gn > 0:
                w.learning_rate = self.base[w.name] * min(max(scale * wn / gn, 0.0), 1e4)


@register("custom_learning_rate")
class CustomLearningRate(_LRSchedule):
    """Placeholder schedule the user overrides from Python via ``schedule`` attribute."""
    schedule = None

    def global_schedule(self, model):
        return float(self.schedule(model)) if self.schedule else 1.0


@register("step_minibatch")
class StepMinibatch(ExecCallback):
    """Grow the mini-batch size by ``step`` every ``ramp_time`` epochs
    (src/callbacks/variable_minibatch.cpp)."""

    def setup(self, model):
        self.current = int(self.params.starting_mbsize)

    def on_train_begin(self, model):
        model.trainer.data_coordinator.set_mini_batch_size("training", self.current)

    def on_epoch_end(self, model):
        ramp = int(self.params.ramp_time) or 1
        if (model.ctx.epoch + 1) % ramp == 0:
            new = min(self.current + int(self.params.step), model.trainer.max_mini_batch_size)
            if new != self.current:
                ratio = new / self.current
                self.current = new
                model.trainer.data_coordinator.set_mini_batch_size("training", new)
                for w in select_weights(model, ""):
                    w.learning_rate = w.learning_rate * ratio


@register("minibatch_schedule")
class MinibatchSchedule(ExecCallback):
    """Explicit (epoch, mbsize, lr, ramp_time) schedule (src/callbacks/variable_minibatch.cpp)."""

    def on_train_begin(self, model):
        model.trainer.data_coordinator.set_mini_batch_size("training", int(self.params.starting_mbsize))

    def on_epoch_end(self, model):
        for s in self.params.step:
            if int(s.epoch) == model.ctx.epoch + 1:
                model.trainer.data_coordinator.set_mini_batch_size(
                    "training", min(int(s.mbsize), model.trainer.max_mini_batch_size))
                if s.lr:
                    for w in select_weights(model, ""):
                        w.learning_rate = float(s.lr)


# =============================================================================== gradients
@register("clip_gradient_norm")
class ClipGradientNorm(ExecCallback):
    """Clip per-weights or global gradient norm (src/callbacks/gradient_clipping.cpp:253)."""

    def setup(self, model):
        self.weights = select_weights(model, getattr(self.params, "weights", ""))

    def on_backward_prop_end(self, model):
        limit = float(self.params.value) or 1.0
        if self.params.global_norm:
            if len(self.weights) == len([w for w in model.weights if w.has_optimizer()]):
                sq = model.arena.grad_sqnorm()
            else:
                sq = sum((w.gradient.float() ** 2).sum() for w in self.weights if w.gradient is not None)
                sq = sq.reshape(1)
            if model.parallel is not None and model.parallel.grads_are_sharded:
                model.parallel.allreduce_sum_inplace(sq)
            scale = torch.clamp(limit / (sq.sqrt() + 1e-12), max=1.0)
            for w in self.weights:
                if w.gradient is not None:
                    w.gradient.mul_(scale.to(w.gradient.dtype))
        else:
            for w in self.weights:
                if w.gradient is None:
                    continue
                n = w.gradient.float().norm()
                w.gradient.mul_(torch.clamp(limit / (n + 1e-12), max=1.0).to(w.gradient.dtype))


@register("check_gradients")
class CheckGradients(ExecCallback):
    """Compare analytic gradients with 4th-order central finite differences of the
    objective (src/callbacks/check_gradients.cpp:121-200,284-300)."""

    def __init__(self, params=None):
        super().__init__(params)
        self.done = False

    def on_test_end(self, model):
        modes = (self.params.execution_modes or "").split()
        if not modes or "test" in modes or "testing" in modes:
            self.run(model, "testing")

    def on_epoch_end(self, model):
        if "training" in (self.params.execution_modes or "").split():
            self.run(model, "training")

    def run(self, model, mode):
        if self.done:
            return
        self.done = True
        inputs = model.trainer.data_coordinator.peek_batch(mode)
        if inputs is None:
            inputs = model.trainer.data_coordinator.peek_batch("training")

        def objective():
            with torch.no_grad():
                model.forward_prop(inputs, "validation")
                v = model.local_objective().double()
                if model.parallel is not None and model.parallel.dp_size > 1:
                    v = v.reshape(1).clone()
                    model.parallel.allreduce_sum_inplace(v)
                return float(v) + float(model.l2_value())

        gen_state = model.generator().get_state()
        model.clear_gradients()
        model.forward_prop(inputs, "validation")
        obj = model.local_objective()
        amp, model.amp_enabled = model.amp_enabled, False
        model.backward_prop(obj)
        model.amp_enabled = amp
        f0 = objective()
        eps = float(torch.finfo(torch.float32).eps)
        step = float(self.params.step_size) or max(abs(f0), 1.0) * eps ** 0.2 * 2
        expected_err = max(eps ** 0.9 * abs(f0) / step, eps ** 0.9) * 1e2 + step ** 4 * 1e2
        worst, failed = 0.0, []
        for w in model.weights:
            if not w.has_optimizer() or w.gradient is None:
                continue
            flat = w.values.detach().view(-1)
            g = w.gradient.view(-1).double()
            if w.slot.l2:
                g = g + w.slot.l2 * flat.double()
            n = flat.numel()
            probe = sorted(set([0, n // 2, n - 1] + [int(i) for i in torch.randint(0, n, (2,)).tolist()]))
            for i in probe:
                old = float(flat[i])
                vals = []
                for k in (2, 1, -1, -2):
                    flat[i] = old + k * step
                    model.arena.refresh_compute()
                    w.handle.bump()
                    model.generator().set_state(gen_state)
                    vals.append(objective())
                flat[i] = old
                model.arena.refresh_compute()
                w.handle.bump()
                fd = (-vals[0] + 8 * vals[1] - 8 * vals[2] + vals[3]) / (12 * step)
                err = abs(fd - float(g[i]))
                rel = err / max(abs(fd), abs(float(g[i])), 1e-12)
                worst = max(worst, err)
                if err > expected_err and rel > 1e-2:
                    failed.append((w.name, i, float(g[i]), fd))
                if self.params.verbose and is_master(model):
                    print(f"  {w.name}[{i}]: analytic {float(g[i]):.6e} numeric {fd:.6e} err {err:.3e}")
        if is_master(model):
            print(f"CHECK GRADIENTS: objective {f0:.6g}, step {step:.3e}, max error {worst:.3e}, "
                  f"{len(failed)} failures", flush=True)
        if failed and self.params.error_on_failure:
            raise RuntimeError(f"gradient check failed: {failed[:5]}")


@register("check_metric")
class CheckMetric(ExecCallback):
    """Assert a metric lies within bounds (src/callbacks/check_metric.cpp)."""

    def _check(self, model, mode):
        modes = (self.params.execution_modes or "").split()
        alias = {"test": "testing", "train": "training"}
        modes = [alias.get(m, m) for m in modes]
        if modes and mode not in modes:
            return
        _, mets, samples = model.reduce_statistics(mode)
        if samples == 0:
            return
        for met, v in zip(model.metrics, mets):
            if met.name == self.params.metric:
                lo, hi = float(self.params.lower_bound), float(self.params.upper_bound)
                ok = lo <= v <= hi and not math.isnan(v)
                if not ok:
                    msg = (f"metric \"{met.name}\" has value {v} which is outside [{lo}, {hi}] "
                           f"during {mode}")
                    if self.params.error_on_failure:
                        raise RuntimeError(msg)
                    if is_master(model):
                        print("WARNING: " + msg, flush=True)
                return
        raise RuntimeError(f"check_metric: no metric named '{self.params.metric}'")

    def on_epoch_end(self, model): self._check(model, "training")
    def on_validation_end(self, model): self._check(model, "validation")
    def on_test_end(self, model): self._check(model, "testing")


@register("check_nan")
class CheckNaN(ExecCallback):
    """Fail on non-finite activations, gradients or weights (src/callbacks/check_nan.cpp)."""

    def on_forward_prop_end(self, model, mode):
        for name, outs in model.acts.items():
            for t in outs:
                if t.is_floating_point() and not bool(torch.isfinite(t).all()):
                    raise RuntimeError(f"check_nan: non-finite activation in layer '{name}' "
                                       f"(step {model.ctx.step})")

    def on_backward_prop_end(self, model):
        for w in model.weights:
            if w.gradient is not None and not bool(torch.isfinite(w.gradient).all()):
                raise RuntimeError(f"check_nan: non-finite gradient for weights '{w.name}'")

    def on_batch_end(self, model):
        for w in model.weights:
            if not bool(torch.isfinite(w.values).all()):
                raise RuntimeError(f"check_nan: non-finite values in weights '{w.name}'")


@register("check_small")
class CheckSmall(ExecCallback):
    """Fail on denormal-range activations / gradients / weights (src/callbacks/check_small.cpp)."""

    def _chk(self, t, what):
        lim = math.sqrt(float(torch.finfo(torch.float32).tiny))
        a = t.detach().float().abs()
        if bool(((a > 0) & (a < lim)).any()):
            raise RuntimeError(f"check_small: {what} has entries below {lim:.3e}")

    def on_forward_prop_end(self, model, mode):
        for name, outs in model.acts.items():
            for t in outs:
                if t.is_floating_point():
                    self._chk(t, f"activation of layer '{name}'")

    def on_backward_prop_end(self, model):
        for w in model.weights:
            if w.gradient is not None:
                self._chk(w.gradient, f"gradient of weights '{w.name}'")

    def on_batch_end(self, model):
        for w in model.weights:
            self._chk(w.values, f"weights '{w.name}'")


@register("check_init", "init")
class CheckInit(ExecCallback):
    """All ranks of a trainer start from identical weights (src/callbacks/check_init.cpp)."""

    def on_train_begin(self, model):
        if model.comm is None or model.comm.procs_per_trainer == 1:
            return
        for w in model.weights:
            v = w.values.detach().float().reshape(-1)
            ref = v.clone()
            model.comm.trainer_broadcast(ref, 0)
            if not torch.equal(ref, v):
                raise RuntimeError(f"check_init: weights '{w.name}' differ across ranks")


@register("check_dataset")
class CheckDataset(ExecCallback):
    """Every training sample is seen exactly once per epoch (src/callbacks/check_dataset.cpp)."""

    def on_epoch_begin(self, model):
        self.seen = []

    def on_batch_end(self, model):
        self.seen.extend(int(i) for i in model.trainer.data_coordinator.last_indices("training"))

    def on_epoch_end(self, model):
        seen = self.seen
        if model.comm is not None:
            seen = [i for part in model.comm.trainer_gather_object(seen) for i in part]
        if is_trainer_master(model):
            n = model.trainer.data_coordinator.num_samples("training")
            if len(seen) != len(set(seen)):
                raise RuntimeError("check_dataset: a sample was processed more than once")
            if len(seen) > n:
                raise RuntimeError("check_dataset: more samples processed than the data set holds")
            print(f"check_dataset: epoch {model.ctx.epoch} processed {len(seen)} of {n} samples", flush=True)


@register("early_stopping")
class EarlyStopping(ExecCallback):
    """Stop when the validation objective has not improved for ``patience`` epochs
    (src/callbacks/early_stopping.cpp)."""

    def setup(self, model):
        self.best, self.wait = float("inf"), 0

    def on_validation_end(self, model):
        obj, _, n = model.reduce_statistics("validation")
        if n == 0:
            return
        if obj < self.best:
            self.best, self.wait = obj, 0
        else:
            self.wait += 1
            if self.wait >= (int(self.params.patience) or 1):
                model.ctx.stop_training = True
                if is_master(model):
                    print(f"{model.name}: early stopping at epoch {model.ctx.epoch}", flush=True)


@register("evaluate_progress")
class EvaluateProgress(ExecCallback):
    """Periodically evaluate on the tournament / validation set during training
    (src/callbacks/evaluate_progress.cpp)."""

    def on_batch_end(self, model):
        if model.ctx.step == 0 or model.ctx.step % self.batch_interval:
            return
        tr = model.trainer
        mode = "tournament" if tr.data_coordinator.num_samples("tournament") else "validation"
        if tr.data_coordinator.num_samples(mode) == 0:
            return
        tr.evaluate(model, mode, report=False)
        obj, mets, _ = model.reduce_statistics(mode)
        if is_trainer_master(model):
            vals = dict(zip([m.name for m in model.metrics], mets))
            pick = vals.get(self.params.metric, obj)
            print(f"{model.name} (instance {_trainer_rank(model)}) step {model.ctx.step} "
                  f"{mode} {self.params.metric or 'objective function'} : {pick:.6g}", flush=True)


@register("confusion_matrix")
class ConfusionMatrix(ExecCallback):
    """Accumulate prediction-vs-label counts and write them as CSV per mode
    (src/callbacks/confusion_matrix.cpp)."""

    def setup(self, model):
        self.counts = {}

    def _acc(self, model, mode):
        pred = model.acts[self.params.prediction][0]
        lab = model.acts[self.params.label][0]
        n = pred.shape[0]
        p = pred.reshape(n, -1).argmax(1)
        l = lab.reshape(n, -1)
        l = l.argmax(1) if l.shape[1] > 1 else l[:, 0].long()
        c = pred.reshape(n, -1).shape[1]
        m = self.counts.setdefault(mode, torch.zeros(c, c, dtype=torch.int64, device=pred.device))
        m.view(-1).index_add_(0, l * c + p, torch.ones_like(p, dtype=torch.int64))

    def _flush(self, model, mode):
        if mode not in self.counts:
            return
        m = self.counts.pop(mode).float()
        if model.parallel is not None and model.parallel.dp_size > 1:
            model.parallel.allreduce_sum_inplace(m)
        if is_trainer_master(model):
            import numpy as np
            tot = max(float(m.sum()), 1.0)
            np.savetxt(f"{self.params.prefix}{mode}-epoch{model.ctx.epoch}.csv",
                       (m / tot).cpu().numpy(), delimiter=",")

    def on_batch_end(self, model): self._acc(model, "training")
    def on_batch_evaluate_end(self, model, mode): self._acc(model, mode)
    def on_epoch_end(self, model): self._flush(model, "training")
    def on_validation_end(self, model): self._flush(model, "validation")
    def on_test_end(self, model): self._flush(model, "testing")
