"""LTFB ("let a thousand flowers bloom") population training and its meta-learning
strategies.

Algorithm (src/execution_algorithms/ltfb.cpp:44-98): repeat {train locally with the inner
algorithm; run the meta-learning strategy} until the tournament budget is spent.
Strategies: random pairwise exchange (ltfb/random_pairwise_exchange.cpp:217-356: partners
drawn from a generator shared by all trainers, both evaluate both models on the tournament
set, the local model survives if it is better on ANY metric), truncation selection
(truncation_selection_exchange.cpp) and regularized evolution (regularized_evolution.cpp),
with model exchange by direct weight transfer (sendrecv_weights.cpp:74-173), in-memory
checkpoint (checkpoint_binary.cpp) or checkpoint files (checkpoint_file.cpp), and optional
mutation (mutation_strategy.cpp).  Models travel between trainers as one flat buffer per
arena over the inter-trainer communicator (rank i of trainer A talks to rank i of B).
"""
from __future__ import annotations

import io
import os
import random
from typing import Dict, List, Optional

import numpy as np
import torch

from ..proto import lbann_pb2 as pb
from .algorithms import ExecutionContext, SGDTrainingAlgorithm, Termination, TrainingAlgorithm

LOWER_IS_BETTER, HIGHER_IS_BETTER = 0, 1


# ------------------------------------------------------------------ model <-> flat state
def pack_model(model, weights_names=None, with_optimizer=True) -> Dict[str, torch.Tensor]:
    out = {}
    names = set(weights_names) if weights_names else None
    if with_optimizer and hasattr(model, "sync_optimizer_state"):
        model.sync_optimizer_state()     # collective over the trainer when the state is sharded
    for w in model.weights:
        if names is not None and w.name not in names:
            continue
        out[f"{w.name}/values"] = w.values.detach().clone()
        if with_optimizer:
            for k, t in w.optimizer_state().items():
                out[f"{w.name}/{k}"] = t.detach().clone()
            out[f"{w.name}/hp"] = torch.tensor(
                [float(w.slot.hp.get(k, 0.0)) for k in ("learn_rate", "momentum", "beta1", "beta2", "eps")],
                dtype=torch.float64)
    return out


def unpack_model(model, state: Dict[str, torch.Tensor], with_optimizer=True):
    for w in model.weights:
        key = f"{w.name}/values"
        if key not in state:
            continue
        w.set_values(state[key].to(model.device))
        if with_optimizer:
            for k, t in w.optimizer_state().items():
                if f"{w.name}/{k}" in state:
                    t.copy_(state[f"{w.name}/{k}"].to(t.device))
            hp = state.get(f"{w.name}/hp")
            if hp is not None:
                for k, v in zip(("learn_rate", "momentum", "beta1", "beta2", "eps"), hp.tolist()):
                    if k in w.slot.hp:
                        w.slot.hp[k] = v
    model.arena.commit_state()           # state kept for the owned blocks only: take this rank's share
    model.arena.refresh_compute()


def exchange_with_partner(trainer, model, partner_trainer: int, strategy: str = "sendrecv_weights",
                          weights_names=None, exchange_hyperparameters=True, checkpoint_dir=None,
                          step: int = 0) -> Dict[str, torch.Tensor]:
    """Send this trainer's model to ``partner_trainer`` and return the partner's."""
    comm = trainer.comm
    mine = pack_model(model, weights_names, exchange_hyperparameters)
    if partner_trainer == comm.trainer_rank:
        return mine
    peer = partner_trainer * comm.procs_per_trainer + comm.rank_in_trainer
    if strategy == "checkpoint_file":
        d = os.path.join(checkpoint_dir or ".", f"ltfb_step{step}")
        os.makedirs(d, exist_ok=True)
        if comm.am_trainer_master():
            torch.save({k: v.cpu() for k, v in mine.items()}, os.path.join(d, f"trainer{comm.trainer_rank}.pt"))
        comm.global_barrier()
        return torch.load(os.path.join(d, f"trainer{partner_trainer}.pt"), map_location=model.device)
    if strategy == "checkpoint_binary":
        bio = io.BytesIO()
        torch.save({k: v.cpu() for k, v in mine.items()}, bio)
        payload = torch.frombuffer(bytearray(bio.getvalue()), dtype=torch.uint8).to(model.device)
        n_mine = torch.tensor([payload.numel()], dtype=torch.int64, device=model.device)
        n_peer = torch.zeros_like(n_mine)
        comm.sendrecv(n_mine, n_peer, peer)
        recv = torch.empty(int(n_peer.item()), dtype=torch.uint8, device=model.device)
        comm.sendrecv(payload, recv, peer)
        return torch.load(io.BytesIO(recv.cpu().numpy().tobytes()), map_location=model.device)
    # sendrecv_weights: one flat fp32 buffer, identical layout on both sides
    keys = sorted(mine)
    flat = torch.cat([mine[k].reshape(-1).to(torch.float64 if k.endswith("/hp") else torch.float32).float()
                      for k in keys])
    recv = torch.empty_like(flat)
    comm.sendrecv(flat, recv, peer)
    out, off = {}, 0
    for k in keys:
        n = mine[k].numel()
        out[k] = recv[off:off + n].reshape(mine[k].shape).to(mine[k].dtype)
        off += n
    return out


def evaluate_metrics(trainer, model, mode="tournament") -> Dict[str, float]:
    dc = trainer.data_coordinator
    if dc.num_samples(mode) == 0:
        mode = "validation" if dc.num_samples("validation") else "testing"
    if dc.num_samples(mode) == 0:
        mode = "training"
        SGDTrainingAlgorithm("eval").evaluate(trainer, model, mode, report=False, max_batches=4)
    else:
        SGDTrainingAlgorithm("eval").evaluate(trainer, model, mode, report=False)
    obj, mets, _ = model.reduce_statistics(mode)
    vals = {m.name: v for m, v in zip(model.metrics, mets)}
    vals["objective function"] = obj
    return vals


# ------------------------------------------------------------------ mutation
class Mutation:
    """null / replace_activation / replace_convolution / hybrid (mutation_strategy.cpp)."""

    ACTS = ["relu", "leaky_relu", "elu"]

    def __init__(self, kind="null_mutation", seed=0):
        self.kind = kind
        self.rng = random.Random(seed)

    def mutate(self, model, step):
        if self.kind in ("replace_activation", "hybrid_mutation"):
            acts = [l for l in model.layers if l.type in self.ACTS and not getattr(l, "fused_into_parent", False)]
            if acts:
                l = self.rng.choice(acts)
                new = self.rng.choice([a for a in self.ACTS if a != l.type] or self.ACTS)
                from .layers_core import Elu, LeakyRelu, Relu
                cls = {"relu": Relu, "leaky_relu": LeakyRelu, "elu": Elu}[new]
                l.__class__ = cls
                l.op = cls.op
                l.type = new
                l.params = getattr(pb.Layer, {"relu": "Relu", "leaky_relu": "LeakyRelu", "elu": "Elu"}[new])()
        if self.kind in ("replace_convolution", "hybrid_mutation"):
            convs = [l for l in model.layers if l.type == "convolution" and
                     all(k == 3 for k in l.ksize) and l.cin == l.cout]
            if convs:
                # re-initialise one same-shape convolution kernel (structure is preserved)
                l = self.rng.choice(convs)
                w = l.w
                with torch.no_grad():
                    fresh = w._initial_values(self.rng.randrange(1 << 30)).reshape(w.values.shape)
                w.set_values(fresh.to(model.device))


# ------------------------------------------------------------------ strategies
class MetaLearningStrategy:
    def select_next(self, trainer, model, ctx):
        raise NotImplementedError


def _better(mine: float, theirs: float, direction: int) -> bool:
    return mine <= theirs if direction == LOWER_IS_BETTER else mine >= theirs


class RandomPairwiseExchange(MetaLearningStrategy):
    def __init__(self, metric_strategies: Dict[str, int], exchange="checkpoint_binary",
                 weights_names=None, exchange_hyperparameters=True, checkpoint_dir=None,
                 mutation: Optional[Mutation] = None, seed=20220106):
        self.metric_strategies = dict(metric_strategies)
        self.exchange = exchange
        self.weights_names = list(weights_names or [])
        self.exchange_hp = exchange_hyperparameters
        self.checkpoint_dir = checkpoint_dir
        self.mutation = mutation or Mutation()
        self.rng = random.Random(seed)     # same sequence on every trainer
        self.step = 0
        self.history: List[dict] = []

    def partner(self, comm) -> int:
        order = list(range(comm.num_trainers))
        self.rng.shuffle(order)
        pos = order.index(comm.trainer_rank)
        mate = pos + 1 if pos % 2 == 0 else pos - 1
        return order[mate] if 0 <= mate < len(order) else comm.trainer_rank

    def select_next(self, trainer, model, ctx):
        comm = trainer.comm
        self.step += 1
        partner = self.partner(comm)
        if partner == comm.trainer_rank:
            return
        local_state = pack_model(model, self.weights_names, True)
        local = evaluate_metrics(trainer, model)
        remote_state = exchange_with_partner(trainer, model, partner, self.exchange,
                                             self.weights_names, self.exchange_hp,
                                             self.checkpoint_dir, self.step)
        unpack_model(model, remote_state, self.exchange_hp)
        remote = evaluate_metrics(trainer, model)
        keep_local = any(_better(local[m], remote[m], d) for m, d in self.metric_strategies.items()
                         if m in local)
        if not self.metric_strategies:
            keep_local = local["objective function"] <= remote["objective function"]
        if keep_local:
            unpack_model(model, local_state, True)
        else:
            self.mutation.mutate(model, self.step)
        self.history.append({"step": self.step, "partner": partner, "kept_local": keep_local,
                             "local": local, "remote": remote})
        if comm.am_trainer_master():
            print(f"LTFB tournament {self.step}: trainer {comm.trainer_rank} vs {partner} -> "
                  f"{'keeps its model' if keep_local else 'adopts the partner model'}", flush=True)


class TruncationSelectionExchange(MetaLearningStrategy):
    """The worst trainers copy a model from the top ``truncation_k``."""

    def __init__(self, metric_strategies, truncation_k=1, seed=20220106):
        self.metric, self.direction = next(iter(metric_strategies.items()))
        self.k = max(int(truncation_k), 1)
        self.rng = random.Random(seed)
        self.step = 0

    def select_next(self, trainer, model, ctx):
        comm = trainer.comm
        self.step += 1
        score = evaluate_metrics(trainer, model)[self.metric]
        scores = comm.intertrainer_gather_object(score)
        scores = comm.broadcast_object(scores, 0, "trainer")
        order = sorted(range(len(scores)), key=lambda i: scores[i],
                       reverse=self.direction == HIGHER_IS_BETTER)
        top = order[:self.k]
        src_of = {t: (t if t in top else top[self.rng.randrange(len(top))]) for t in range(len(scores))}
        me = comm.trainer_rank
        for dst, src in sorted(src_of.items()):
            if dst == src:
                continue
            if me == src:
                state = pack_model(model)
                keys = sorted(state)
                flat = torch.cat([state[k].reshape(-1).float() for k in keys])
                comm.send(flat, dst * comm.procs_per_trainer + comm.rank_in_trainer)
            elif me == dst:
                state = pack_model(model)
                keys = sorted(state)
                flat = torch.empty(sum(state[k].numel() for k in keys), dtype=torch.float32,
                                   device=model.device)
                comm.recv(flat, src * comm.procs_per_trainer + comm.rank_in_trainer)
                off = 0
                for k in keys:
                    n = state[k].numel()
                    state[k] = flat[off:off + n].reshape(state[k].shape).to(state[k].dtype)
                    off += n
                unpack_model(model, state)


class RegularizedEvolution(MetaLearningStrategy):
    """Sample a subset of trainers, the best of the sample becomes the parent of the oldest
    trainer's replacement, which is then mutated."""

    def __init__(self, metric_name, metric_strategy, mutation: Optional[Mutation] = None,
                 sample_size=0, seed=20220106):
        self.metric, self.direction = metric_name, metric_strategy
        self.mutation = mutation or Mutation()
        self.sample_size = sample_size
        self.rng = random.Random(seed)
        self.age: Optional[List[int]] = None
        self.step = 0

    def select_next(self, trainer, model, ctx):
        comm = trainer.comm
        n = comm.num_trainers
        self.step += 1
        if self.age is None:
            self.age = [0] * n
        self.age = [a + 1 for a in self.age]
        score = evaluate_metrics(trainer, model)[self.metric]
        scores = comm.broadcast_object(comm.intertrainer_gather_object(score), 0, "trainer")
        sample = self.rng.sample(range(n), min(self.sample_size or n, n))
        parent = (max if self.direction == HIGHER_IS_BETTER else min)(sample, key=lambda i: scores[i])
        oldest = max(range(n), key=lambda i: self.age[i])
        if oldest != parent:
            helper = TruncationSelectionExchange({self.metric: self.direction}, 1)
            me = comm.trainer_rank
            if me == parent:
                state = pack_model(model)
                flat = torch.cat([state[k].reshape(-1).float() for k in sorted(state)])
                comm.send(flat, oldest * comm.procs_per_trainer + comm.rank_in_trainer)
            elif me == oldest:
                state = pack_model(model)
                keys = sorted(state)
                flat = torch.empty(sum(state[k].numel() for k in keys), dtype=torch.float32,
                                   device=model.device)
                comm.recv(flat, parent * comm.procs_per_trainer + comm.rank_in_trainer)
                off = 0
                for k in keys:
                    m = state[k].numel()
                    state[k] = flat[off:off + m].reshape(state[k].shape).to(state[k].dtype)
                    off += m
                unpack_model(model, state)
                self.mutation.mutate(model, self.step)
            del helper
        self.age[oldest] = 0


def build_strategy(any_msg) -> MetaLearningStrategy:
    name = any_msg.type_url.split(".")[-1]
    if name == "RandomPairwiseExchange":
        m = pb.RandomPairwiseExchange()
        any_msg.Unpack(m)
        es = m.exchange_strategy
        kind = es.WhichOneof("strategy") or "checkpoint_binary"
        return RandomPairwiseExchange(
            dict(m.metric_name_strategy_map), kind, list(es.weights_name),
            bool(es.sendrecv_weights.exchange_hyperparameters) if kind == "sendrecv_weights" else True,
            es.checkpoint_file.checkpoint_dir if kind == "checkpoint_file" else None,
            Mutation(m.mutation_strategy.WhichOneof("strategy") or "null_mutation"))
    if name == "TruncationSelectionExchange":
        m = pb.TruncationSelectionExchange()
        any_msg.Unpack(m)
        return TruncationSelectionExchange(dict(m.metric_name_strategy_map), int(m.truncation_k))
    if name == "RegularizedEvolution":
        m = pb.RegularizedEvolution()
        any_msg.Unpack(m)
        return RegularizedEvolution(m.metric_name, int(m.metric_strategy),
                                    Mutation(m.mutation_strategy.WhichOneof("strategy") or "null_mutation"),
                                    int(m.sample_size))
    raise ValueError(f"unknown meta-learning strategy '{name}'")


class LTFB(TrainingAlgorithm):
    def __init__(self, name, local_algo: SGDTrainingAlgorithm, strategy: MetaLearningStrategy,
                 max_tournaments: int = 1):
        self.name = name
        self.local = local_algo
        self.strategy = strategy
        self.max_tournaments = max_tournaments

    def apply(self, trainer, model, ctx: ExecutionContext, mode="training"):
        if mode != "training":
            return self.local.evaluate(trainer, model, mode)
        base = self.local.termination
        for t in range(self.max_tournaments):
            # the inner criteria are per round: extend them from the current position
            term = Termination(max_epochs=(ctx.epoch + base.max_epochs) if base.max_epochs else 0,
                               max_batches=(ctx.step + base.max_batches) if base.max_batches else 0,
                               max_seconds=base.max_seconds)
            self.local.train(trainer, model, ctx, term)
            ctx.stop_training = False
            self.strategy.select_next(trainer, model, ctx)
