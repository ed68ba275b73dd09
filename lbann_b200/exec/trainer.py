"""Trainer: owns the communicator, the data coordinator, trainer-level callbacks, the
training algorithm and execution contexts; builds models from an ``LbannPB`` experiment.

Counterpart of src/trainers/trainer.cpp and the construction helpers of
src/utils/lbann_library.cpp:144-537 (seeds, readers, I/O threads, model build).
"""
from __future__ import annotations

import os
import time
from typing import Dict, Optional

import torch

from ..callbacks import build_callback
from ..data.coordinator import DataCoordinator
from ..data.readers import build_reader
from ..parallel.comm import LbannComm
from ..proto import lbann_pb2 as pb
from ..utils import options as opts
from .algorithms import ExecutionContext, SGDTrainingAlgorithm, Termination, build_training_algorithm
from .model import ExecModel

_DT = {"float": torch.float32, "fp32": torch.float32, "bf16": torch.bfloat16,
       "bfloat16": torch.bfloat16, "fp16": torch.float16, "half": torch.float16,
       "float16": torch.float16, "double": torch.float64}


def pick_device(comm_local_rank: int = 0, disable_cuda: bool = False) -> torch.device:
    if not disable_cuda and torch.cuda.is_available():
        dev = torch.device("cuda", comm_local_rank % torch.cuda.device_count())
        torch.cuda.set_device(dev)
        return dev
    return torch.device("cpu")


class ExecTrainer:
    def __init__(self, lbann_pb, *, comm: Optional[LbannComm] = None, device=None,
                 default_dtype=None, procs_per_trainer: int = 0, grid_height: int = 0,
                 io_threads: Optional[int] = None, background_io: Optional[bool] = None,
                 readers: Optional[Dict] = None):
        self.proto = lbann_pb
        tp = lbann_pb.trainer
        self.name = tp.name or "trainer"
        o = opts.current()
        disable_cuda = bool(lbann_pb.model.disable_cuda) or o.get_bool("disable_cuda")
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.device = torch.device(device) if device is not None else pick_device(local_rank, disable_cuda)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            # run (and first-touch pinned buffers) on the cores next to this GPU
            from ..utils.affinity import bind_to_gpu
            self.cpu_binding = bind_to_gpu(self.device.index if self.device.index is not None else 0)
        self.comm = comm or LbannComm(procs_per_trainer or o.get_int("procs_per_trainer"),
                                      grid_height or o.get_int("trainer_grid_height") or 1,
                                      device=self.device)
        if self.comm.num_trainers > 1:
            self.name = f"{self.name}{self.comm.trainer_rank}" if tp.name else f"trainer{self.comm.trainer_rank}"
        dt = default_dtype or o.get("default_dtype") or ("bf16" if False else "float")
        self.default_dtype = _DT[dt] if isinstance(dt, str) else dt
        seed = int(tp.random_seed) or o.get_int("random_seed") or 42
        # trainers start from different seeds unless asked otherwise (lbann_library.cpp:228-267)
        identical = bool(tp.random_init_trainers_identically) or o.get_bool("random_init_models_identically")
        self.seed = seed if identical else seed + 1000 * self.comm.trainer_rank
        self.data_seed = seed
        torch.manual_seed(self.seed + 7 * self.comm.rank_in_trainer)
        self.max_mini_batch_size = int(tp.mini_batch_size) or o.get_int("mini_batch_size") or 1
        self.callbacks = [build_callback(c) for c in tp.callback]
        self.contexts: Dict[tuple, ExecutionContext] = {}
        self.last_timing = {}
        self.timer_sync = False
        self.models = []
        self.io_threads = io_threads if io_threads is not None else (o.get_int("num_io_threads") or 2)
        from ..utils.random import init_random
        init_random(self.data_seed, self.comm.rank_in_world, self.comm.rank_in_trainer,
                    self.comm.trainer_rank, self.io_threads)
        self.background_io = (not bool(tp.serialize_io)) if background_io is None else background_io
        if o.get_bool("serialize_io") or o.get_bool("disable_background_io_activity"):
            self.background_io = False
        if "omp_num_threads" in o._values or o._env("omp_num_threads"):   # only when asked for
            torch.set_num_threads(max(1, o.get_int("omp_num_threads")))
        self.parallel = None
        self.distconv = None
        self._readers_override = readers
        self.data_coordinator: Optional[DataCoordinator] = None
        self.algorithm = None
        self.persist = None
        for cb in self.callbacks:
            cb.setup_trainer(self)

    # ---------------------------------------------------------------- construction
    def _build_readers(self):
        if self._readers_override is not None:
            readers = dict(self._readers_override)
            for r in readers.values():
                if not len(r.indices):
                    r.setup(self.data_seed)
            return readers
        readers = {}
        for rp in self.proto.data_reader.reader:
            md = self.proto.data_set_metadata if self.proto.HasField("data_set_metadata") else None
            r = build_reader(rp, md)
            r.setup(self.data_seed)
            readers[r.role] = r
        tr = readers.get("train")
        if tr is not None:
            for role, frac in (("validate", tr.validation_fraction), ("tournament", tr.tournament_fraction)):
                if frac > 0 and role not in readers:
                    import copy
                    part = tr.split(frac)
                    clone = copy.copy(tr)
                    clone.role = role
                    clone.indices = part
                    clone.shuffle = False
                    readers[role] = clone
        return readers

    def setup_parallel(self, model_pb):
        """Create the data-/tensor-/spatial-parallel contexts when more than one rank
        participates in the trainer."""
        if self.comm.procs_per_trainer > 1:
            from ..parallel.context import ParallelContext
            self.parallel = ParallelContext(self.comm, self.device)
        n_sub = opts.current().get_int("num_subgrids") or opts.current().get_int("num_subgrids_block_order")
        if self.parallel is not None and n_sub > 1:
            # branch (sub-graph) parallelism: layers tagged with a grid run on that GPU subset
            from ..parallel.subgrid import SubgridContext
            self.parallel.subgrid = SubgridContext(self.comm, self.device, n_sub, self.parallel.group)
            self.parallel._subgrids = True
        def partitions(l):      # a strategy that only names a grid is not a tensor partition
            ps = l.parallel_strategy
            return any(getattr(ps, f, 0) for f in ("sample_groups", "depth_groups", "height_groups",
                                                   "width_groups", "channel_groups", "filter_groups"))
        needs_dc = any(l.HasField("parallel_strategy") and partitions(l) for l in model_pb.layer)
        if needs_dc and not opts.current().get_bool("disable_distconv"):
            from ..parallel.distconv import DistconvContext
            self.distconv = DistconvContext(self.comm, self.device, self.parallel)
            self.distconv.plan(model_pb)

    def build_model(self, model_pb=None) -> ExecModel:
        model_pb = model_pb if model_pb is not None else self.proto.model
        if self.parallel is None and self.distconv is None:
            self.setup_parallel(model_pb)
        if self.data_coordinator is None:
            readers = self._build_readers()
            dp_rank, dp_size = 0, 1
            if self.parallel is not None:
                dp_rank, dp_size = self.parallel.data_rank(self.distconv), self.parallel.data_size(self.distconv)
            o = opts.current()
            if o.get_bool("use_data_store") or o.get_bool("preload_data_store"):
                from ..data.store import DataStore
                pg = DataStore.make_group() if dp_size == self.comm.world_size and dp_size > 1 else None
                world = dp_size if (pg is not None or dp_size == 1) else 1
                for k, role in enumerate(sorted(readers)):
                    spill = str(o.get("data_store_spill", "") or "")
                    sdir = os.path.join(spill, role) if spill else ""
                    warm = bool(sdir) and os.path.exists(os.path.join(sdir, f"data_store_rank{dp_rank if world > 1 else 0}.npz"))
                    st = DataStore(readers[role], dp_rank if world > 1 else 0, world, pg,
                                   preload=o.get_bool("preload_data_store") and not warm, tag=k)
                    if warm:
                        st.load_spilled(sdir)        # warm cache from an earlier run: no file is read
                    st.spill_dir = sdir
                    readers[role] = st
            self.data_coordinator = DataCoordinator(
                readers, self.max_mini_batch_size, device=self.device, dp_rank=dp_rank,
                dp_size=dp_size, seed=self.data_seed, io_threads=self.io_threads,
                background=self.background_io)
        dc = self.data_coordinator
        allocator = self.parallel.arena_allocator() if self.parallel is not None else None
        model = ExecModel(model_pb, self.proto.optimizer if self.proto.HasField("optimizer") else None,
                          device=self.device, default_dtype=self.default_dtype,
                          data_dims=dc.dims, slice_points=dc.slice_points, comm=self.comm,
                          parallel=self.parallel, distconv=self.distconv, seed=self.seed,
                          arena_allocator=allocator)
        model.trainer = self
        model.ctx = self.context(model, "training")
        model.callbacks = [build_callback(c) for c in model_pb.callback]
        for cb in self.callbacks + model.callbacks:
            cb.on_setup_begin(model)
        model.setup()
        for cb in self.callbacks + model.callbacks:
            cb.setup(model)
        for cb in self.callbacks + model.callbacks:
            cb.on_setup_end(model)
        self.models.append(model)
        if self.algorithm is None:
            algo_pb = self.proto.trainer.training_algorithm if self.proto.trainer.HasField(
                "training_algorithm") else (self.proto.training_algorithm if self.proto.HasField(
                    "training_algorithm") else None)
            self.algorithm = build_training_algorithm(algo_pb, model.num_epochs)
        return model

    def context(self, model, mode) -> ExecutionContext:
        key = (id(model), "training" if mode == "training" else mode)
        if key not in self.contexts:
            self.contexts[key] = ExecutionContext(mode)
        return self.contexts[key]

    # ---------------------------------------------------------------- running
    def train(self, model: ExecModel, num_epochs: Optional[int] = None, num_batches: int = 0):
        ctx = self.context(model, "training")
        model.ctx = ctx
        algo = self.algorithm
        if num_epochs is not None or num_batches:
            base = algo if isinstance(algo, SGDTrainingAlgorithm) else None
            if base is not None:
                base.termination = Termination(max_epochs=num_epochs or 0, max_batches=num_batches)
        algo.apply(self, model, ctx, "training")

    def evaluate(self, model: ExecModel, mode: str = "testing", report: bool = True, max_batches: int = 0):
        algo = self.algorithm if isinstance(self.algorithm, SGDTrainingAlgorithm) else \
            SGDTrainingAlgorithm("sgd")
        if getattr(model, "ctx", None) is None:
            model.ctx = self.context(model, "training")
        algo.evaluate(self, model, mode, report, max_batches)

    def shutdown(self):
        if hasattr(self.algorithm, "shutdown"):
            self.algorithm.shutdown()
        if self.data_coordinator is not None:
            for st in self.data_coordinator.modes.values():
                r = getattr(st, "reader", None)
                if getattr(r, "spill_dir", "") and hasattr(r, "spill"):
                    r.spill(r.spill_dir)
            self.data_coordinator.shutdown()
