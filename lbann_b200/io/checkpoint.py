"""Checkpoint / restart in the reference's directory layout.

    <checkpoint_dir>/<trainer_name>/
        sgd.last.shared.checkpoint              "hook=<hook> epoch=E step=S"
        sgd.shared.<hook>.epoch.E.step.S/
            <model_name>/model.bin              weights, optimizer state and hyper-parameters
            trainer.bin                         mini-batch size, seeds, background-I/O flag
            training_ctx.bin validation_ctx.bin testing_ctx.bin ...
            rng_state/rng_generator_<rank>      host and device generator states
            data_coordinator.bin                reader positions and shuffled indices
        sgd.last.distributed.checkpoint
        sgd.rank.R.distributed.<hook>.epoch.E.step.S/ ...   (every rank writes its own)

(src/callbacks/checkpoint.cpp:106-298,549-833, src/models/model.cpp:2093-2195,
src/trainers/trainer.cpp:333-352, src/utils/random.cpp:41-157.)  The files are tensor
containers (io/container.py) rather than cereal archives; names and placement are the
reference's.  ``shared`` checkpoints are written by the trainer master; weights sharded
over ranks are gathered first.
"""
from __future__ import annotations

import os
import re
import time
from typing import Optional, Tuple

import numpy as np
import torch

from . import container

ALGO = "sgd"


def trainer_dir(base: str, trainer_name: str) -> str:
    return os.path.join(base, trainer_name)


def shared_dir(base, trainer_name, hook, epoch, step) -> str:
    return os.path.join(trainer_dir(base, trainer_name), f"{ALGO}.shared.{hook}.epoch.{epoch}.step.{step}")


def distributed_dir(base, trainer_name, rank, hook, epoch, step) -> str:
    return os.path.join(trainer_dir(base, trainer_name),
                        f"{ALGO}.rank.{rank}.distributed.{hook}.epoch.{epoch}.step.{step}")


def latest_file(base, trainer_name, kind="shared") -> str:
    return os.path.join(trainer_dir(base, trainer_name), f"{ALGO}.last.{kind}.checkpoint")


def write_latest(base, trainer_name, kind, hook, epoch, step):
    os.makedirs(trainer_dir(base, trainer_name), exist_ok=True)
    tmp = latest_file(base, trainer_name, kind) + ".tmp"
    with open(tmp, "w") as f:
        f.write(f"hook={hook} epoch={epoch} step={step}\n")
    os.replace(tmp, latest_file(base, trainer_name, kind))


def read_latest(base, trainer_name, kind="shared") -> Optional[Tuple[str, int, int]]:
    path = latest_file(base, trainer_name, kind)
    if not os.path.exists(path):
        return None
    m = re.match(r"hook=(\S+) epoch=(\d+) step=(\d+)", open(path).read())
    return (m.group(1), int(m.group(2)), int(m.group(3))) if m else None


# ------------------------------------------------------------------ model / trainer payloads
def model_state(model, gather_sharded: bool = True):
    # optimizer state that is sharded over the trainer's ranks is made whole first (collective)
    if hasattr(model, "sync_optimizer_state"):
        model.sync_optimizer_state()
    tensors, meta = {}, {"name": model.name, "weights": {}, "amp_scale": model.amp_scale}
    if getattr(model, "_amp_state", None) is not None:
        # loss scale, its inverse, clean steps, consecutive skipped steps, last step's inverse
        meta["amp_state"] = [float(v) for v in model._amp_state.tolist()]
    else:
        meta["amp_counters"] = [int(getattr(model, "_amp_good_steps", 0)),
                                int(getattr(model, "_amp_skipped", 0))]
    for w in model.weights:
        vals = w.values.detach()
        if getattr(w, "export_values", None) is not None:
            vals = w.export_values()         # the layer keeps the live copy elsewhere
        elif gather_sharded and model.parallel is not None and getattr(w, "shard", None) is not None:
            vals = model.parallel.gather_sharded_weights(w)
        tensors[f"weights/{w.name}/values"] = vals.float().cpu()
        for k, t in w.optimizer_state().items():
            tensors[f"weights/{w.name}/{k}"] = t.detach().float().cpu()
        meta["weights"][w.name] = {"shape": list(w.shape), "optimizer": w.slot.kind,
                                   "hyperparameters": {k: float(v) if not isinstance(v, bool) else v
                                                       for k, v in w.slot.hp.items()},
                                   "step_count": w.slot.step_count}
    if model.arena.step_dev is not None:
        meta["optimizer_step"] = int(model.arena.step_dev.item())
    return tensors, meta


def load_model_state(model, tensors, meta, strict: bool = True):
    for w in model.weights:
        key = f"weights/{w.name}/values"
        if key not in tensors:
            if strict:
                raise KeyError(f"checkpoint has no weights '{w.name}'")
            continue
        w.set_values(tensors[key].to(model.device))
        if getattr(w, "after_load", None) is not None:
            w.after_load()
        info = meta.get("weights", {}).get(w.name, {})
        if info:
            w.slot.hp.update(info.get("hyperparameters", {}))
            w.slot.step_count = int(info.get("step_count", 0))
        for k, t in w.optimizer_state().items():
            tk = f"weights/{w.name}/{k}"
            if tk in tensors:
                t.copy_(tensors[tk].to(t.device).reshape(t.shape))
    if getattr(model, "arena", None) is not None:
        model.arena.commit_state()       # state kept for the owned blocks only: take this rank's share
    if "optimizer_step" in meta and model.device.type == "cuda":
        a = model.arena
        if a.step_dev is None:
            a.step_dev = torch.zeros(1, dtype=torch.int32, device=model.device)
            a.lr_scale_dev = torch.ones(1, dtype=torch.float32, device=model.device)
        a.step_dev.fill_(int(meta["optimizer_step"]))
    model.amp_scale = float(meta.get("amp_scale", model.amp_scale))
    if "amp_state" in meta and model.device.type == "cuda" and model.amp_enabled:
        st = model._amp_device_state()
        st.copy_(torch.tensor(meta["amp_state"], dtype=torch.float32))
    elif "amp_state" in meta:
        model._amp_good_steps = int(meta["amp_state"][2])
        model._amp_skipped = int(meta["amp_state"][3])
    elif "amp_counters" in meta:
        model._amp_good_steps, model._amp_skipped = (int(v) for v in meta["amp_counters"])
    model.arena.refresh_compute()


def save_model(model, path: str):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    tensors, meta = model_state(model)
    container.save(path, tensors, meta)


def load_model(model, path: str, strict: bool = True):
    tensors, meta = container.load(path)
    load_model_state(model, tensors, meta, strict)


def _save_rng(dirpath: str, rank: int, model):
    os.makedirs(os.path.join(dirpath, "rng_state"), exist_ok=True)
    t = {"torch_cpu": torch.get_rng_state()}
    if model._gen is not None:
        t["model_generator"] = model._gen.get_state().cpu()
    from ..utils.random import banks
    container.save(os.path.join(dirpath, "rng_state", f"rng_generator_{rank}"), t,
                   {"numpy": [str(x) if not isinstance(x, np.ndarray) else x.tolist()
                              for x in np.random.get_state()],
                    # model / fast / data-sequence / LTFB / per-thread I/O generators of this rank
                    "banks": banks().dumps()})


def _load_rng(dirpath: str, rank: int, model):
    path = os.path.join(dirpath, "rng_state", f"rng_generator_{rank}")
    if not os.path.exists(path):
        import warnings
        warnings.warn(f"checkpoint {dirpath} has no random-generator state for rank {rank}: this "
                      "rank continues with fresh random streams, the restart is not reproducible")
        return
    t, meta = container.load(path)
    torch.set_rng_state(t["torch_cpu"])
    if "model_generator" in t:
        model.generator().set_state(t["model_generator"])
    if meta.get("banks"):
        from ..utils.random import banks
        banks().loads(meta["banks"])
    st = meta.get("numpy")
    if st:
        np.random.set_state((st[0], np.asarray(st[1], dtype=np.uint32), int(st[2]), int(st[3]), float(st[4])))


def save_checkpoint(trainer, model, base: str, hook: str, distributed: bool = False,
                    per_rank_base: Optional[str] = None) -> str:
    ctx = trainer.context(model, "training")
    comm = trainer.comm
    rank = comm.rank_in_trainer
    t0 = time.time()
    if distributed:
        d = distributed_dir(per_rank_base or base, trainer.name, rank, hook, ctx.epoch, ctx.step)
        os.makedirs(d, exist_ok=True)
        tensors, meta = model_state(model, gather_sharded=False)
        os.makedirs(os.path.join(d, model.name), exist_ok=True)
        container.save(os.path.join(d, model.name, "model.bin"), tensors, meta)
        write_it = True
    else:
        d = shared_dir(base, trainer.name, hook, ctx.epoch, ctx.step)
        tensors, meta = model_state(model, gather_sharded=True)   # collective when sharded
        write_it = comm.am_trainer_master()
        if write_it:
            os.makedirs(os.path.join(d, model.name), exist_ok=True)
            container.save(os.path.join(d, model.name, "model.bin"), tensors, meta)
    if write_it:
        container.save(os.path.join(d, "trainer.bin"), {}, {
            "max_mini_batch_size": trainer.max_mini_batch_size, "seed": trainer.seed,
            "data_seed": trainer.data_seed, "background_io": bool(trainer.background_io),
            "name": trainer.name})
        for (mid, mode), c in trainer.contexts.items():
            if mid == id(model):
                container.save(os.path.join(d, f"{mode}_ctx.bin"), {}, c.state())
        dc = trainer.data_coordinator.state()
        arrays = {f"{m}/order": torch.from_numpy(s["order"]) for m, s in dc.items()}
        arrays.update({f"{m}/reader_indices": torch.from_numpy(s["reader"]["indices"])
                       for m, s in dc.items() if s["reader"] is not None})
        container.save(os.path.join(d, "data_coordinator.bin"), arrays,
                       {m: {"pos": s["pos"], "epoch": s["epoch"], "mb": s["mb"]} for m, s in dc.items()})
    # every rank keeps its own generators (src/utils/random.cpp save_rng_to_checkpoint writes
    # one file per rank in shared checkpoints too): the master has made the directory by now
    comm.trainer_barrier()
    _save_rng(d, rank, model)
    comm.trainer_barrier()
    if comm.am_trainer_master():
        write_latest(per_rank_base or base if distributed else base, trainer.name,
                     "distributed" if distributed else "shared", hook, ctx.epoch, ctx.step)
        nbytes = sum(t.numel() * t.element_size() for t in tensors.values())
        dt = max(time.time() - t0, 1e-9)
        print(f"[{trainer.name}] Checkpoint [{'distributed' if distributed else 'shared'}]: "
              f"epoch {ctx.epoch} step {ctx.step} in {dt:.3f}s ({nbytes / dt / 2**20:.1f} MiB/s) -> {d}",
              flush=True)
    return d


def find_latest(base: str, trainer_name: str, per_rank_base: Optional[str] = None):
    """(kind, hook, epoch, step) of the newest checkpoint, preferring the later step."""
    s = read_latest(base, trainer_name, "shared")
    d = read_latest(per_rank_base or base, trainer_name, "distributed")
    if s is None and d is None:
        return None
    if d is None or (s is not None and (s[1], s[2]) >= (d[1], d[2])):
        return ("shared",) + s
    return ("distributed",) + d


def restore_checkpoint(trainer, model, base: str, per_rank_base: Optional[str] = None) -> bool:
    comm = trainer.comm
    found = find_latest(base, trainer.name, per_rank_base) if comm.am_trainer_master() else None
    found = comm.broadcast_object(found, 0, "trainer")
    if found is None:
        return False
    kind, hook, epoch, step = found
    if kind == "shared":
        d = shared_dir(base, trainer.name, hook, epoch, step)
    else:
        d = distributed_dir(per_rank_base or base, trainer.name, comm.rank_in_trainer, hook, epoch, step)
    tensors, meta = container.load(os.path.join(d, model.name, "model.bin"))
    if kind == "shared" and model.parallel is not None:
        tensors = model.parallel.scatter_loaded_weights(model, tensors)
    load_model_state(model, tensors, meta)
    for (mid, mode), c in list(trainer.contexts.items()) + [((id(model), "training"), trainer.context(model, "training"))]:
        p = os.path.join(d, f"{mode}_ctx.bin")
        if mid == id(model) and os.path.exists(p):
            c.load_state(container.load(p)[1])
    p = os.path.join(d, "data_coordinator.bin")
    if os.path.exists(p):
        arrays, m = container.load(p)
        state = {}
        for mode, s in m.items():
            state[mode] = {"pos": s["pos"], "epoch": s["epoch"], "mb": s["mb"],
                           "order": arrays[f"{mode}/order"].numpy(),
                           "reader": ({"indices": arrays[f"{mode}/reader_indices"].numpy()}
                                      if f"{mode}/reader_indices" in arrays else None)}
        trainer.data_coordinator.load_state(state)
    _load_rng(d, comm.rank_in_trainer, model)
    ctx = trainer.context(model, "training")
    st = trainer.data_coordinator.modes["training"]
    # resume inside an epoch only when the checkpoint was taken inside one (a position at
    # the end of the sample order means the epoch had finished)
    ctx._resume_mid_epoch = 0 < st.pos < len(st.order)
    if comm.am_trainer_master():
        print(f"[{trainer.name}] Restart from {kind} checkpoint: hook {hook} epoch {epoch} step {step}",
              flush=True)
    return True
