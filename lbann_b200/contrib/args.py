"""Command-line helpers for application scripts (python/lbann/contrib/args.py:12-369)."""
from __future__ import annotations

import argparse

from ..frontend import core as L


def add_scheduler_arguments(parser: argparse.ArgumentParser, default_job_name: str = "lbann"):
    g = parser.add_argument_group("launcher")
    g.add_argument("--nodes", type=int, default=1, help="number of compute nodes")
    g.add_argument("--procs-per-node", type=int, default=None, help="processes (GPUs) per node")
    g.add_argument("--partition", default=None)
    g.add_argument("--account", default=None)
    g.add_argument("--reservation", default=None)
    g.add_argument("--time-limit", type=int, default=None, help="minutes")
    g.add_argument("--job-name", default=default_job_name)
    g.add_argument("--work-dir", default=None)
    g.add_argument("--batch-job", action="store_true", help="submit instead of running now")
    g.add_argument("--setup-only", action="store_true", help="write the experiment, do not run")


def get_scheduler_kwargs(args) -> dict:
    kw = {}
    for src, dst in (("nodes", "nodes"), ("procs_per_node", "procs_per_node"), ("partition", "partition"),
                     ("account", "account"), ("reservation", "reservation"), ("time_limit", "time_limit"),
                     ("job_name", "job_name"), ("work_dir", "work_dir"), ("batch_job", "batch_job"),
                     ("setup_only", "setup_only")):
        v = getattr(args, src, None)
        if v not in (None, False):
            kw[dst] = v
    return kw


def get_distconv_environment(parallel_io: bool = False, num_io_partitions: int = 1) -> dict:
    """Environment of a distconv run: halo exchange and shuffles over peer memory."""
    env = {"LBANN_DISTCONV_HALO_EXCHANGE": "P2P", "LBANN_DISTCONV_TENSOR_SHUFFLER": "P2P",
           "LBANN_DISTCONV_RANK_STRIDE": "1", "LBANN_KEEP_ERROR_SIGNALS": "1"}
    if parallel_io:
        env["LBANN_DISTCONV_NUM_IO_PARTITIONS"] = str(num_io_partitions)
    return env


def add_optimizer_arguments(parser, default_optimizer="momentum", default_learning_rate=0.01):
    g = parser.add_argument_group("optimizer")
    g.add_argument("--optimizer", default=default_optimizer,
                   choices=["momentum", "sgd", "adam", "adagrad", "rmsprop"])
    g.add_argument("--optimizer-learning-rate", type=float, default=default_learning_rate)


def create_optimizer(args):
    lr = args.optimizer_learning_rate
    return {"momentum": lambda: L.SGD(learn_rate=lr, momentum=0.9),
            "sgd": lambda: L.SGD(learn_rate=lr),
            "adam": lambda: L.Adam(learn_rate=lr, beta1=0.9, beta2=0.99, eps=1e-8),
            "adagrad": lambda: L.AdaGrad(learn_rate=lr, eps=1e-8),
            "rmsprop": lambda: L.RMSprop(learn_rate=lr, decay_rate=0.99, eps=1e-8)}[args.optimizer]()


def add_profiling_arguments(parser) -> None:
    g = parser.add_argument_group("profiling")
    g.add_argument("--profile", action="store_true", help="time every layer (CallbackTimer + summary)")
    g.add_argument("--profile-init", action="store_true")
    g.add_argument("--caliper", action="store_true", help="accepted for compatibility; not used")


def create_profile_callbacks(args):
    cbs = []
    if getattr(args, "profile", False):
        cbs.append(L.CallbackProfiler(skip_init=not getattr(args, "profile_init", False)))
    return cbs


def get_profile_args(args):
    return ["--layer_timing"] if getattr(args, "profile", False) else []


def add_training_arguments(parser, default_minibatch_size=256, default_epochs=10) -> None:
    g = parser.add_argument_group("training")
    g.add_argument("--mini-batch-size", type=int, default=default_minibatch_size)
    g.add_argument("--num-epochs", type=int, default=default_epochs)
    g.add_argument("--random-seed", type=int, default=None)


def add_amp_arguments(parser) -> None:
    g = parser.add_argument_group("mixed precision")
    g.add_argument("--amp", action="store_true", help="16-bit layers with dynamic loss scaling")
    g.add_argument("--amp-init-scale", type=float, default=None)
