"""Checkpointing, dumps, summaries, weight manipulation and population-training callbacks.

Each class names the reference source it mirrors (src/callbacks/*.cpp).
"""
from __future__ import annotations

import math
import os
import struct
import time
import zlib

import numpy as np
import torch

from ..io import checkpoint as ckpt
from .base import (ExecCallback, is_master, is_trainer_master, register, select_layers,
                   select_weights)


def _rank(model):
    return model.comm.rank_in_world if model.comm is not None else 0


def _trainer_name(model):
    return model.trainer.name


# =============================================================================== checkpointing
@register("checkpoint")
class Checkpoint(ExecCallback):
    """Shared / distributed checkpoints by epoch, step or wall-clock interval and restart
    from ``restart_dir`` (src/callbacks/checkpoint.cpp:87-298)."""

    def __init__(self, params=None):
        super().__init__(params)
        p = params
        self.dir = p.checkpoint_dir
        self.restart_dir = p.restart_dir or p.checkpoint_dir
        self.epochs, self.steps, self.secs = int(p.checkpoint_epochs), int(p.checkpoint_steps), float(p.checkpoint_secs)
        self.per_rank_dir = p.per_rank_dir or None
        self.dist_epochs, self.dist_steps = int(p.ckpt_dist_epochs), int(p.ckpt_dist_steps)
        self.last_time = time.time()
        self.restored = False

    def on_train_begin(self, model):
        if self.restart_dir and not self.restored:
            self.restored = True
            ckpt.restore_checkpoint(model.trainer, model, self.restart_dir, self.per_rank_dir)
        self.last_time = time.time()

    def _maybe(self, model, hook, epoch_boundary):
        ctx = model.ctx
        if not self.dir:
            return
        shared = dist = False
        if epoch_boundary:
            shared = self.epochs > 0 and ctx.epoch > 0 and ctx.epoch % self.epochs == 0
            dist = self.dist_epochs > 0 and ctx.epoch > 0 and ctx.epoch % self.dist_epochs == 0
        else:
            shared = self.steps > 0 and ctx.step > 0 and ctx.step % self.steps == 0
            dist = self.dist_steps > 0 and ctx.step > 0 and ctx.step % self.dist_steps == 0
            if self.secs > 0:
                due = time.time() - self.last_time >= self.secs
                if model.comm is not None:
                    due = model.comm.broadcast_object(due, 0, "trainer")
                shared = shared or due
        if shared:
            ckpt.save_checkpoint(model.trainer, model, self.dir, hook, False)
            self.last_time = time.time()
        if dist:
            ckpt.save_checkpoint(model.trainer, model, self.dir, hook, True, self.per_rank_dir)

    def on_epoch_begin(self, model):
        self._maybe(model, "epoch_begin", True)

    def on_batch_begin(self, model):
        self._maybe(model, "training_batch_begin", False)

    def on_train_end(self, model):
        if self.dir and (self.epochs or self.steps or self.secs):
            ckpt.save_checkpoint(model.trainer, model, self.dir, "training_end", False)


@register("save_model")
class SaveModel(ExecCallback):
    """Write the model's weights after training (src/callbacks/save_model.cpp:111-160)."""

    def on_train_end(self, model):
        if self.params.disable_save_after_training:
            return
        self.save(model)

    def save(self, model):
        d = os.path.join(self.params.dir, _trainer_name(model), model.name)
        tensors, meta = ckpt.model_state(model)
        if is_trainer_master(model):
            os.makedirs(d, exist_ok=True)
            from ..io import container
            container.save(os.path.join(d, "model.bin"), tensors, meta)
            for w in model.weights:
                v = tensors[f"weights/{w.name}/values"]
                h = v.shape[0] if v.dim() else 1
                wd = v.numel() // max(h, 1)
                v.numpy().astype(np.float32).tofile(os.path.join(d, f"model_weights_{w.name}_{h}x{wd}.bin"))
            with open(os.path.join(self.params.dir, _trainer_name(model), "last_saved_model"), "w") as f:
                f.write(d + "\n")


@register("load_model")
class LoadModel(ExecCallback):
    """Load weights from ``model.bin`` or per-weights files before training
    (src/callbacks/load_model.cpp:59-205)."""

    def on_setup_end(self, model):
        for d in (self.params.dirs or "").split():
            cands = [os.path.join(d, model.name, "model.bin"), os.path.join(d, "model.bin")]
            hit = next((c for c in cands if os.path.exists(c)), None)
            if hit:
                ckpt.load_model(model, hit, strict=False)
                if is_master(model):
                    print(f"load_model: loaded {hit}", flush=True)
                return
            found = 0
            for w in model.weights:
                for fn in os.listdir(d) if os.path.isdir(d) else []:
                    if fn.startswith(f"model_weights_{w.name}_") and fn.endswith(".bin"):
                        arr = np.fromfile(os.path.join(d, fn), dtype=np.float32)
                        w.set_values(torch.from_numpy(arr).to(model.device))
                        found += 1
            if found:
                return
        raise RuntimeError(f"load_model: no model found in '{self.params.dirs}'")


@register("dump_weights")
class DumpWeights(ExecCallback):
    """Weights to text / binary / npy files every ``epoch_interval`` epochs
    (src/callbacks/dump_weights.cpp)."""

    def _dump(self, model, tag):
        if not is_trainer_master(model):
            return
        d = os.path.join(self.params.directory or ".", _trainer_name(model), model.name)
        os.makedirs(d, exist_ok=True)
        fmt = (self.params.format or "text").lower()
        for w in model.weights:
            a = w.values.detach().float().cpu().numpy()
            base = os.path.join(d, f"{tag}-{w.name}-Weights")
            if fmt in ("npy", "distributed_binary") or fmt == "numpy":
                np.save(base + ".npy", a)
            elif fmt == "binary":
                a.tofile(base + ".bin")
            else:
                np.savetxt(base + ".txt", a.reshape(a.shape[0], -1) if a.ndim else a.reshape(1, 1))

    def on_train_begin(self, model):
        self._dump(model, "initial")

    def on_epoch_end(self, model):
        iv = int(self.params.epoch_interval) or 1
        if (model.ctx.epoch + 1) % iv == 0:
            self._dump(model, f"epoch{model.ctx.epoch + 1}")


@register("dump_outputs")
class DumpOutputs(ExecCallback):
    """Layer outputs per step to
    ``<dir>/<trainer>/<model>/sgd.<mode>.epoch.E.step.S_<layer>_output<k>.<ext>``
    (src/callbacks/dump_outputs.cpp; the naming is relied on by ``lbann.evaluate``)."""

    def _dump(self, model, mode):
        modes = (self.params.execution_modes or "").split()
        alias = {"test": "testing", "train": "training", "validate": "validation"}
        if modes and mode not in [alias.get(m, m) for m in modes]:
            return
        ctx = model.ctx
        step = ctx.step - 1 if mode == "training" else getattr(ctx, "eval_step", 0)
        if self.batch_interval > 1 and step % self.batch_interval:
            return
        d = os.path.join(self.params.directory or ".", _trainer_name(model), model.name)
        os.makedirs(d, exist_ok=True)
        fmt = (self.params.format or "csv").lower()
        names = (self.params.layers or "").split() or [l.name for l in model.layers]
        epoch = ctx.epoch
        for name in names:
            for k, t in enumerate(model.acts.get(name, [])):
                a = t.detach().float().cpu().numpy()
                if model.comm is not None and model.comm.procs_per_trainer > 1 and model.parallel is not None:
                    parts = model.comm.trainer_gather_object(a)
                    a = model.parallel.interleave_samples(parts)
                if not is_trainer_master(model):
                    continue
                base = os.path.join(d, f"sgd.{mode}.epoch.{epoch}.step.{max(step, 0)}_{name}_output{k}")
                flat = a.reshape(a.shape[0], -1)
                if fmt == "npy":
                    np.save(base + ".npy", flat)
                elif fmt == "npz":
                    np.savez(base + ".npz", data=flat)
                else:
                    np.savetxt(base + (".tsv" if fmt == "tsv" else ".csv"), flat,
                               delimiter="\t" if fmt == "tsv" else ",")

    def on_batch_end(self, model): self._dump(model, "training")

    def on_batch_evaluate_end(self, model, mode):
        model.ctx.eval_step = getattr(model.ctx, "eval_step", -1) + 1
        self._dump(model, mode)

    def on_validation_begin(self, model): model.ctx.eval_step = -1
    def on_test_begin(self, model): model.ctx.eval_step = -1


@register("dump_gradients")
class DumpGradients(ExecCallback):
    """src/callbacks/dump_gradients.cpp"""

    def on_backward_prop_end(self, model):
        iv = int(self.params.interval) or 1
        if model.ctx.step % iv:
            return
        base = self.params.basename or "gradients"
        for w in model.weights:
            if w.gradient is not None and is_trainer_master(model):
                np.savetxt(f"{base}model0-epoch{model.ctx.epoch}-step{model.ctx.step}-{w.name}-Gradient.txt",
                           w.gradient.float().cpu().numpy().reshape(-1))


@register("dump_error_signals")
class DumpErrorSignals(ExecCallback):
    """Gradients w.r.t. every layer output (src/callbacks/dump_error_signals.cpp); captured
    with autograd hooks on the activations."""

    def on_forward_prop_end(self, model, mode):
        if mode != "training":
            return
        base = self.params.basename or ""
        step, epoch = model.ctx.step, model.ctx.epoch
        for name, outs in model.acts.items():
            for k, t in enumerate(outs):
                if t.requires_grad:
                    def hook(g, name=name, k=k):
                        np.savetxt(f"{base}model0-epoch{epoch}-step{step}-{name}-ErrorSignal{k}.txt",
                                   g.detach().float().cpu().numpy().reshape(g.shape[0], -1))
                    t.register_hook(hook)


@register("dump_mb_indices")
class DumpMinibatchSampleIndices(ExecCallback):
    """src/callbacks/dump_minibatch_sample_indices.cpp"""

    def on_batch_end(self, model):
        iv = int(self.params.interval) or 1
        if (model.ctx.step - 1) % iv:
            return
        idx = model.trainer.data_coordinator.last_indices("training")
        base = self.params.basename or ""
        with open(f"{base}model0-training-epoch{model.ctx.epoch}-step{model.ctx.step - 1}-"
                  f"r{_rank(model)}-MB_Sample_Indices.txt", "w") as f:
            f.write("\n".join(str(int(i)) for i in idx) + "\n")


@register("dump_model_graph")
class DumpModelGraph(ExecCallback):
    """Graphviz description of the layer graph (src/callbacks/dump_model_graph.cpp)."""

    def on_setup_end(self, model):
        if not is_master(model):
            return
        lines = ["digraph G {"]
        for l in model.layers:
            lines.append(f'  "{l.name}" [label="{l.name}\\n{l.type} {list(l.out_dims)}"];')
            for c in l.child_names:
                lines.append(f'  "{l.name}" -> "{c}";')
        lines.append("}")
        text = "\n".join(lines)
        with open((self.params.basename or "model_graph") + ".dot", "w") as f:
            f.write(text + "\n")
        if self.params.print:
            print(text, flush=True)


# =============================================================================== TensorBoard
_CRC_TABLE = None


def _crc32c(data: bytes) -> int:
    global _CRC_TABLE
    if _CRC_TABLE is None:
        tbl = []
        for i in range(256):
            c = i
            for _ in range(8):
                c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
            tbl.append(c)
        _CRC_TABLE = tbl
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked(data: bytes) -> int:
    c = _crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


class EventWriter:
    """Minimal TensorFlow event-file writer (scalars, histograms, PNG images): the role of
    the reference's external/TBinf library and src/utils/summary.cpp."""

    def __init__(self, logdir: str):
        os.makedirs(logdir, exist_ok=True)
        self.path = os.path.join(logdir, f"events.out.tfevents.{int(time.time())}.lbann")
        self.f = open(self.path, "ab")
        self._record(_field(1, 1, struct.pack("<d", time.time())) +
                     _field(3, 2, _varint(len(b"brain.Event:2")) + b"brain.Event:2"))

    def _record(self, event: bytes):
        hdr = struct.pack("<Q", len(event))
        self.f.write(hdr + struct.pack("<I", _masked(hdr)) + event + struct.pack("<I", _masked(event)))
        self.f.flush()

    def _event(self, step: int, value: bytes):
        summary = _field(1, 2, _varint(len(value)) + value)
        self._record(_field(1, 1, struct.pack("<d", time.time())) + _field(2, 0, _varint(step)) +
                     _field(5, 2, _varint(len(summary)) + summary))

    def scalar(self, tag: str, value: float, step: int):
        t = tag.encode()
        self._event(step, _field(1, 2, _varint(len(t)) + t) + _field(2, 5, struct.pack("<f", float(value))))

    def histogram(self, tag: str, values: np.ndarray, step: int, bins: int = 30):
        v = np.asarray(values, dtype=np.float64).reshape(-1)
        if v.size == 0:
            return
        counts, edges = np.histogram(v, bins=bins)
        h = (_field(1, 1, struct.pack("<d", v.min())) + _field(2, 1, struct.pack("<d", v.max())) +
             _field(3, 1, struct.pack("<d", float(v.size))) + _field(4, 1, struct.pack("<d", v.sum())) +
             _field(5, 1, struct.pack("<d", float((v * v).sum()))))
        lim = b"".join(struct.pack("<d", e) for e in edges[1:])
        cnt = b"".join(struct.pack("<d", float(c)) for c in counts)
        h += _field(6, 2, _varint(len(lim)) + lim) + _field(7, 2, _varint(len(cnt)) + cnt)
        t = tag.encode()
        self._event(step, _field(1, 2, _varint(len(t)) + t) + _field(5, 2, _varint(len(h)) + h))

    def image(self, tag: str, chw: np.ndarray, step: int):
        png = encode_png(chw)
        c, h, w = chw.shape
        img = (_field(1, 0, _varint(h)) + _field(2, 0, _varint(w)) + _field(3, 0, _varint(c)) +
               _field(4, 2, _varint(len(png)) + png))
        t = tag.encode()
        self._event(step, _field(1, 2, _varint(len(t)) + t) + _field(4, 2, _varint(len(img)) + img))

    def close(self):
        self.f.close()


def encode_png(chw: np.ndarray) -> bytes:
    """8-bit PNG (grey / RGB) from a [C, H, W] float array in [0, 1]."""
    a = np.clip(np.asarray(chw, dtype=np.float32), 0, 1)
    if a.ndim == 2:
        a = a[None]
    c, h, w = a.shape
    if c not in (1, 3):
        a, c = a[:1], 1
    img = (a.transpose(1, 2, 0) * 255 + 0.5).astype(np.uint8)
    raw = b"".join(b"\x00" + img[r].tobytes() for r in range(h))

    def chunk(kind, data):
        body = kind + data
        return struct.pack(">I", len(data)) + body + struct.pack(">I", zlib.crc32(body) & 0xFFFFFFFF)
    ihdr = struct.pack(">IIBBBBB", w, h, 8, 0 if c == 1 else 2, 0, 0, 0)
    return b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", ihdr) + chunk(b"IDAT", zlib.compress(raw)) + chunk(b"IEND", b"")


def _summarizer(model):
    sw = getattr(model, "_summary_writer", None)
    if sw is None and is_master(model):
        d = model.proto.summarizer.dir if model.proto.HasField("summarizer") else ""
        if d:
            sw = model._summary_writer = EventWriter(d)
    return sw


@register("summary")
class Summary(ExecCallback):
    """Objective, metrics, timings and weight histograms to TensorBoard
    (src/callbacks/summary.cpp)."""

    def on_batch_end(self, model):
        sw = _summarizer(model)
        bi = int(self.params.batch_interval) or 0
        if sw is None or not bi or model.ctx.step % bi:
            return
        sw.scalar("objective", float(model.last_objective), model.ctx.step)
        mi = int(self.params.mat_interval) or 0
        if mi and model.ctx.step % mi == 0:
            for w in model.weights:
                sw.histogram(f"weights/{w.name}", w.values.detach().float().cpu().numpy(), model.ctx.step)

    def on_epoch_end(self, model):
        obj, mets, _ = model.reduce_statistics("training")
        sw = _summarizer(model)
        if sw is None:
            return
        sw.scalar("objective/train_epoch", obj, model.ctx.epoch)
        for m, v in zip(model.metrics, mets):
            sw.scalar(f"{m.name}/train_epoch", v, model.ctx.epoch)
        for l in model.layers:
            if l.fp_time:
                sw.scalar(f"fp_time/{l.name}", l.fp_time, model.ctx.epoch)

    def on_test_end(self, model):
        obj, mets, _ = model.reduce_statistics("testing")
        sw = _summarizer(model)
        if sw is None:
            return
        sw.scalar("objective/test", obj, model.ctx.epoch)
        for m, v in zip(model.metrics, mets):
            sw.scalar(f"{m.name}/test", v, model.ctx.epoch)


@register("summarize_images")
class SummarizeImages(ExecCallback):
    """Selected validation images to TensorBoard (src/callbacks/summarize_images.cpp)."""

    def on_batch_evaluate_end(self, model, mode):
        sw = _summarizer(model)
        iv = int(self.params.epoch_interval) or 1
        if sw is None or model.ctx.epoch % iv:
            return
        name = self.params.image_source_layer_name
        if name not in model.acts:
            return
        imgs = model.acts[name][0].detach().float().cpu().numpy()
        strat = self.params.selection_strategy
        limit = 10
        if strat.HasField("categorical_accuracy"):
            limit = int(strat.categorical_accuracy.num_images) or 10
        elif strat.HasField("track_sample_ids"):
            limit = int(strat.track_sample_ids.num_tracked_images) or 10
        for i in range(min(limit, imgs.shape[0])):
            a = imgs[i]
            a = (a - a.min()) / max(a.max() - a.min(), 1e-12)
            sw.image(f"{name}/sample{i}", a if a.ndim == 3 else a.reshape(1, *a.shape[-2:]), model.ctx.epoch)


@register("save_images")
class SaveImages(ExecCallback):
    """Layer outputs as image files each epoch (src/callbacks/save_images.cpp)."""

    def on_epoch_end(self, model):
        if not is_trainer_master(model):
            return
        for name in (self.params.layers or "").split():
            if name not in model.acts:
                continue
            a = model.acts[name][0][0].detach().float().cpu().numpy()
            if a.ndim == 1:
                s = int(math.sqrt(a.size))
                a = a[:s * s].reshape(1, s, s)
            a = (a - a.min()) / max(a.max() - a.min(), 1e-12)
            ext = self.params.image_format or "png"
            with open(f"{self.params.image_prefix}epoch{model.ctx.epoch}-{name}.{ext}", "wb") as f:
                f.write(encode_png(a))


@register("save_topk_models")
class SaveTopKModels(ExecCallback):
    """Across trainers, the k best by a metric save their model
    (src/callbacks/save_topk_models.cpp)."""

    def on_test_end(self, model):
        _, mets, _ = model.reduce_statistics("testing")
        vals = dict(zip([m.name for m in model.metrics], mets))
        if self.params.metric not in vals:
            raise RuntimeError(f"save_topk_models: no metric '{self.params.metric}'")
        score = vals[self.params.metric]
        scores = model.comm.intertrainer_gather_object(score) if model.comm is not None else [score]
        scores = model.comm.broadcast_object(scores, 0, "trainer") if model.comm is not None else scores
        order = sorted(range(len(scores)), key=lambda i: scores[i], reverse=not self.params.ascending_ordering)
        me = model.comm.trainer_rank if model.comm is not None else 0
        if me in order[:max(int(self.params.k), 1)]:
            p = type("P", (), {"dir": self.params.dir, "disable_save_after_training": False})
            SaveModel(p).save(model)


@register("export_onnx")
class ExportOnnx(ExecCallback):
    """Writes the trained model as an ONNX file (binary ``ModelProto``, opset 11) to
    ``output_filename`` (default ``lbann.onnx``); ``debug_string_filename`` receives the text
    form of the same message (src/callbacks/export_onnx.cpp).  The graph is built by
    ``io/onnx_export.py``; the ``onnx`` package is not needed."""

    def on_train_end(self, model):
        if not is_master(model):
            return
        from google.protobuf import text_format
        from ..io.onnx_export import export_model
        mp = export_model(model)
        with open(self.params.output_filename or "lbann.onnx", "wb") as f:
            f.write(mp.SerializeToString())
        if self.params.debug_string_filename:
            for t in mp.graph.initializer:          # values are in the binary file; keep the text readable
                t.raw_data = b""
            with open(self.params.debug_string_filename, "w") as f:
                f.write(text_format.MessageToString(mp))


# =============================================================================== weights manipulation
@register("replace_weights")
class ReplaceWeights(ExecCallback):
    """Copy weights of source layers into destination layers every ``batch_interval`` steps
    (src/callbacks/replace_weights.cpp)."""

    def on_batch_end(self, model):
        if model.ctx.step % self.batch_interval:
            return
        src = (self.params.source_layers or "").split()
        dst = (self.params.destination_layers or "").split()
        for s, d in zip(src, dst):
            for ws, wd in zip(model.layers_by_name[s].weights, model.layers_by_name[d].weights):
                if ws is not None and wd is not None:
                    wd.set_values(ws.values.detach())


@register("set_weights_value")
class SetWeightsValue(ExecCallback):
    """src/callbacks/set_weights_value.cpp"""

    def on_batch_begin(self, model):
        if model.ctx.step == int(self.params.step):
            w = model.weights_by_name[self.params.weights]
            w.set_values(torch.full(w.shape or (1,), float(self.params.value), device=model.device))


def _perturb(value, factor, rng, lo=None, hi=None):
    if factor == 0:
        return value
    v = value * math.exp(rng.normal(0.0, factor)) if value != 0 else rng.normal(0.0, factor)
    if lo is not None:
        v = max(v, lo)
    if hi is not None:
        v = min(v, hi)
    return v


class _Perturb(ExecCallback):
    def setup(self, model):
        seed = (model.trainer.seed * 31 + 7) % (2 ** 31 - 1)
        self.rng = np.random.RandomState(seed)

    def on_setup_end(self, model):
        self.perturb(model)

    def on_batch_begin(self, model):
        during = getattr(self.params, "perturb_during_training", False)
        if during and model.ctx.step > 0 and self.batch_interval and model.ctx.step % self.batch_interval == 0:
            self.perturb(model)


@register("perturb_adam")
class PerturbAdam(_Perturb):
    """Log-normal perturbation of Adam hyper-parameters (population-based training;
    src/callbacks/perturb_adam.cpp)."""

    def perturb(self, model):
        p = self.params
        for w in select_weights(model, p.weights):
            if w.slot.kind != "adam":
                continue
            hp = w.slot.hp
            hp["learn_rate"] = _perturb(hp.get("learn_rate", 0.0), p.learning_rate_factor, self.rng, 0.0)
            hp["beta1"] = 1 - _perturb(1 - hp.get("beta1", 0.9), p.beta1_factor, self.rng, 1e-9, 1.0)
            hp["beta2"] = 1 - _perturb(1 - hp.get("beta2", 0.99), p.beta2_factor, self.rng, 1e-9, 1.0)
            hp["eps"] = _perturb(hp.get("eps", 1e-8), p.eps_factor, self.rng, 0.0)


@register("perturb_learning_rate")
class PerturbLearningRate(_Perturb):
    """src/callbacks/perturb_learning_rate.cpp"""

    def perturb(self, model):
        for w in select_weights(model, self.params.weights):
            w.learning_rate = _perturb(w.learning_rate, self.params.learning_rate_factor, self.rng, 0.0)


@register("perturb_dropout")
class PerturbDropout(_Perturb):
    """src/callbacks/perturb_dropout.cpp"""

    def perturb(self, model):
        for l in select_layers(model, self.params.layers):
            if l.type == "dropout":
                keep = float(l.params.keep_prob) or 0.5
                l.keep_prob_override = _perturb(keep, self.params.keep_dropout_factor, self.rng, 0.05, 1.0)


@register("perturb_weights")
class PerturbWeights(_Perturb):
    """src/callbacks/perturb_weights.cpp"""

    def perturb(self, model):
        p = self.params
        w = model.weights_by_name.get(p.output_name)
        if w is None or self.rng.rand() > (p.perturb_probability or 1.0):
            return
        v = w.values.detach().float()
        noise = torch.from_numpy(self.rng.normal(0, p.scale or 1.0, size=tuple(v.shape)).astype(np.float32))
        w.set_values(torch.clamp(v.cpu() + noise, p.lower or -float("inf"), p.upper or float("inf")))

    def on_batch_begin(self, model):
        if model.ctx.step > 0 and model.ctx.step % self.batch_interval == 0:
            self.perturb(model)


@register("alternate_updates")
class AlternateUpdates(ExecCallback):
    """Alternate between freezing two layer sets, ``iters_1`` / ``iters_2`` steps each (GAN
    training; src/callbacks/alternate_updates.cpp)."""

    def setup(self, model):
        self.sets = [select_layers(model, self.params.layers_1), select_layers(model, self.params.layers_2)]
        self.iters = [int(self.params.iters_1) or 1, int(self.params.iters_2) or 1]
        self.saved = {}

    def _freeze(self, model, layers, frozen):
        for l in layers:
            l.frozen = frozen              # layers without weights (identity_zero) switch on this
            for w in l.weights:
                if w is None or w.slot is None:
                    continue
                if frozen and w.slot.kind != "none":
                    self.saved[w.name] = w.slot.kind
                    w.slot.kind = "none"
                elif not frozen and w.name in self.saved:
                    w.slot.kind = self.saved.pop(w.name)

    def on_batch_begin(self, model):
        period = sum(self.iters)
        phase = 0 if (model.ctx.step % period) < self.iters[0] else 1
        self._freeze(model, self.sets[phase], False)
        self._freeze(model, self.sets[1 - phase], True)


@register("mixup")
class Mixup(ExecCallback):
    """Convex combinations of samples and labels with Beta(alpha, alpha) weights
    (src/callbacks/mixup.cpp)."""

    def on_forward_prop_begin(self, model, mode):
        if mode != "training":
            return
        model._mixup = {"layers": set((self.params.layers or "").split()), "perm": None, "lam": None}

    def on_layer_forward_end(self, model, layer, mode):
        st = getattr(model, "_mixup", None)
        if mode != "training" or st is None or layer.type != "input":
            return
        samples_layer = layer.name in st["layers"]
        is_label = layer.field == "labels"
        if not (samples_layer or is_label):
            return
        t = model.acts[layer.name][0]
        n = t.shape[0]
        if st["perm"] is None:
            a = float(self.params.alpha) or 1.0
            lam = np.random.beta(a, a, size=n).astype(np.float32)
            st["lam"] = torch.from_numpy(np.maximum(lam, 1 - lam)).to(t.device)
            st["perm"] = torch.randperm(n, device=t.device)
        lam = st["lam"].view(n, *([1] * (t.dim() - 1))).to(t.dtype)
        model.acts[layer.name][0] = lam * t + (1 - lam) * t[st["perm"]]


@register("imcomm")
class ImComm(ExecCallback):
    """Average weights / gradients across trainers (src/callbacks/imcomm.cpp)."""

    def on_backward_prop_end(self, model):
        comm = model.comm
        if comm is None or comm.num_trainers == 1:
            return
        for w in model.weights:
            if w.gradient is not None:
                comm.allreduce(w.gradient, "intertrainer")
                w.gradient.div_(comm.num_trainers)


@register("ltfb")
class LegacyLTFB(ExecCallback):
    """Tournament exchange as a callback (src/callbacks/ltfb.cpp, kept for old experiment
    files); delegates to the LTFB training algorithm's exchange logic."""

    def setup(self, model):
        from ..exec.ltfb import RandomPairwiseExchange
        p = self.params
        strat = {"sendrecv_weights": "sendrecv_weights", "checkpoint_file": "checkpoint_file"}.get(
            p.communication_algorithm or "sendrecv_weights", "sendrecv_weights")
        self.strategy = RandomPairwiseExchange(
            {p.metric: (0 if p.low_score_wins else 1)}, strat, (p.weights or "").split(),
            bool(p.exchange_hyperparameters), p.checkpoint_basedir or None)

    def on_batch_begin(self, model):
        if model.ctx.step > 0 and model.ctx.step % self.batch_interval == 0:
            self.strategy.select_next(model.trainer, model, model.ctx)
