"""Execution contexts, termination criteria and training algorithms.

``SGDTrainingAlgorithm`` is the mini-batch loop of the reference
(src/execution_algorithms/sgd_training_algorithm.cpp:99-294,312-393): per step
clear gradients -> forward -> objective -> backward (gradient sync overlapped) -> update,
callbacks honouring ``batch_interval``, validation after each epoch, termination by
epochs / batches / seconds (:533-590).  ``LTFB`` and ``KFAC`` wrap it
(src/execution_algorithms/ltfb.cpp:44-98, kfac.cpp:122).
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from ..proto import lbann_pb2 as pb


class ExecutionContext:
    """Step / epoch counters of one (model, mode) pair (sgd_execution_context.cpp:40-110)."""

    def __init__(self, mode="training"):
        self.mode = mode
        self.step = 0
        self.epoch = 0
        self.step_in_epoch = 0
        self.start_time = time.time()
        self.stop_training = False

    def state(self):
        return {"mode": self.mode, "step": self.step, "epoch": self.epoch}

    def load_state(self, st):
        self.step, self.epoch = int(st["step"]), int(st["epoch"])


class Termination:
    def __init__(self, max_epochs=0, max_batches=0, max_seconds=0.0):
        self.max_epochs, self.max_batches, self.max_seconds = max_epochs, max_batches, max_seconds

    def __call__(self, ctx: ExecutionContext) -> bool:
        if ctx.stop_training:
            return True
        if self.max_epochs and ctx.epoch >= self.max_epochs:
            return True
        if self.max_batches and ctx.step >= self.max_batches:
            return True
        if self.max_seconds and time.time() - ctx.start_time >= self.max_seconds:
            return True
        return not (self.max_epochs or self.max_batches or self.max_seconds)


def _cbs(trainer, model):
    return list(trainer.callbacks) + list(model.callbacks)


class TrainingAlgorithm:
    name = "algorithm"

    def apply(self, trainer, model, ctx: ExecutionContext, mode="training"):
        raise NotImplementedError


class SGDTrainingAlgorithm(TrainingAlgorithm):
    def __init__(self, name="sgd", termination: Optional[Termination] = None,
                 suppress_timer=False):
        self.name = name
        self.termination = termination or Termination()
        self.suppress_timer = suppress_timer

    def apply(self, trainer, model, ctx, mode="training"):
        if mode == "training":
            return self.train(trainer, model, ctx)
        return self.evaluate(trainer, model, mode)

    # ---------------------------------------------------------------- training
    def train(self, trainer, model, ctx, term: Optional[Termination] = None):
        term = term or self.termination
        dc = trainer.data_coordinator
        cbs = _cbs(trainer, model)
        model.ctx = ctx
        ctx.mode = "training"
        ctx.start_time = time.time()
        for cb in cbs:
            cb.on_train_begin(model)
        # hierarchical wall-clock timers, printed at the end of the run with --verbose
        # (src/execution_algorithms/sgd_training_algorithm.cpp:75-96)
        from ..utils.profiling import TimerMap
        timers = self.timers = TimerMap(self.name or "sgd")
        epoch_scope = None
        while not term(ctx):
            if epoch_scope is not None:
                epoch_scope.__exit__(None, None, None)
            epoch_scope = timers.scope("epoch")
            epoch_scope.__enter__()
            model.reset_statistics("training")
            if not getattr(ctx, "_resume_mid_epoch", False):
                dc.start_epoch("training")
                ctx.step_in_epoch = 0
            ctx._resume_mid_epoch = False
            for cb in cbs:
                cb.on_epoch_begin(model)
            finished_epoch = False
            while True:
                batch = dc.next_batch("training")
                if batch is None:
                    finished_epoch = True
                    break
                with timers.scope("mini-batch"):
                    self.train_mini_batch(trainer, model, ctx, batch, cbs)
                if batch.end_of_epoch:
                    finished_epoch = True
                    break
                if (term.max_batches and ctx.step >= term.max_batches) or ctx.stop_training or \
                        (term.max_seconds and time.time() - ctx.start_time >= term.max_seconds):
                    break
            if not finished_epoch:
                ctx._resume_mid_epoch = True
                break
            for cb in cbs:
                cb.on_epoch_end(model)
            ctx.epoch += 1
            if dc.num_samples("validation"):
                self.evaluate(trainer, model, "validation")
        if epoch_scope is not None:
            epoch_scope.__exit__(None, None, None)
        from ..utils import options as _opts
        if _opts.current().get_bool("verbose") and trainer.comm.am_world_master():
            print(timers.report(), flush=True)
        for cb in cbs:
            cb.on_train_end(model)

    def train_mini_batch(self, trainer, model, ctx, batch, cbs):
        for cb in cbs:
            if ctx.step % cb.batch_interval == 0:
                cb.on_batch_begin(model)
        model.train_step(batch.tensors, batch.global_size, batch.offset)
        ctx.step += 1
        ctx.step_in_epoch += 1
        for cb in cbs:
            if (ctx.step - 1) % cb.batch_interval == 0:
                cb.on_batch_end(model)

    # ---------------------------------------------------------------- evaluation
    def evaluate(self, trainer, model, mode, report=True, max_batches=0):
        dc = trainer.data_coordinator
        if dc.num_samples(mode) == 0:
            return
        cbs = _cbs(trainer, model) if report else []
        prev_mode = model.ctx.mode if getattr(model, "ctx", None) is not None else None
        if getattr(model, "ctx", None) is None:
            model.ctx = ExecutionContext(mode)
        model.ctx.mode = mode
        model.reset_statistics(mode)
        begin = {"validation": "on_validation_begin", "testing": "on_test_begin"}.get(mode)
        end = {"validation": "on_validation_end", "testing": "on_test_end"}.get(mode)
        for cb in cbs:
            if begin:
                getattr(cb, begin)(model)
        dc.start_epoch(mode)
        n = 0
        while True:
            batch = dc.next_batch(mode)
            if batch is None:
                break
            for cb in cbs:
                cb.on_batch_evaluate_begin(model, mode)
            model.evaluate_step(batch.tensors, mode, batch.global_size, batch.offset)
            for cb in cbs:
                cb.on_batch_evaluate_end(model, mode)
            n += 1
            if batch.end_of_epoch or (max_batches and n >= max_batches):
                break
        for cb in cbs:
            if end:
                getattr(cb, end)(model)
        if prev_mode is not None:
            model.ctx.mode = prev_mode


class BatchFunctionalInference(TrainingAlgorithm):
    """Forward-only over in-memory samples; returns the arg-max label per sample
    (include/lbann/execution_algorithms/batch_functional_inference_algorithm.hpp)."""
    name = "batch_functional_inference"

    @torch.no_grad()
    def infer(self, model, samples: torch.Tensor, mini_batch_size: int, field="samples",
              output_layer: Optional[str] = None):
        outs = []
        layer = output_layer or model.layers[-1].name
        for i in range(0, samples.shape[0], mini_batch_size):
            x = samples[i:i + mini_batch_size].to(model.device)
            model.forward_prop({field: x}, "prediction")
            y = model.acts[layer][0]
            outs.append(y.reshape(y.shape[0], -1).argmax(1).cpu())
        return torch.cat(outs) if outs else torch.zeros(0, dtype=torch.long)


def build_training_algorithm(algo_pb, default_epochs: int = 0):
    """TrainingAlgorithm message -> algorithm object (src/execution_algorithms/factory.cpp)."""
    if algo_pb is None or not algo_pb.HasField("parameters"):
        return SGDTrainingAlgorithm("sgd", Termination(max_epochs=default_epochs))
    type_name = algo_pb.parameters.type_url.split(".")[-1]
    if type_name == "SGD":
        msg = pb.SGD()
        algo_pb.parameters.Unpack(msg)
        return _sgd_from_msg(algo_pb.name or "sgd", msg, default_epochs)
    if type_name == "LTFB":
        from .ltfb import LTFB, build_strategy
        msg = pb.LTFB()
        algo_pb.parameters.Unpack(msg)
        local = build_training_algorithm(msg.local_training_algorithm, default_epochs)
        return LTFB(algo_pb.name or "ltfb", local, build_strategy(msg.meta_learning_strategy),
                    int(msg.stopping_criteria.max_tournaments) or 1)
    if type_name == "KFAC":
        from .kfac import KFAC
        msg = pb.KFAC()
        algo_pb.parameters.Unpack(msg)
        return KFAC(algo_pb.name or "kfac", _sgd_from_msg("sgd", msg.sgd, default_epochs), msg)
    raise ValueError(f"unknown training algorithm '{type_name}'")


def _sgd_from_msg(name, msg, default_epochs):
    sc = msg.stopping_criteria
    term = Termination(int(sc.max_epochs), int(sc.max_batches), float(sc.max_seconds))
    if not (term.max_epochs or term.max_batches or term.max_seconds):
        term.max_epochs = default_epochs
    return SGDTrainingAlgorithm(name, term, bool(msg.suppress_timer_output))
