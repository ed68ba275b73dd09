"""lbann_b200: a Blackwell-native HPC deep-learning training framework with the user-facing
contract of LBANN (Python front end, prototext schema, trainer / training-algorithm
semantics, callbacks, checkpoint layout) on top of PyTorch, hand-written sm_100a CUDA
kernels and an NVSwitch-native communicator.

``import lbann_b200 as lbann`` gives the model-description API::

    x = lbann.Input(data_field="samples")
    y = lbann.FullyConnected(x, num_neurons=10, has_bias=True)
    ...
    lbann.run(trainer, model, data_reader, optimizer)
"""
from __future__ import annotations

import sys as _sys

from .proto import (callbacks_pb2, data_coordinator_pb2, datatype_pb2, layers_pb2, lbann_pb2,  # noqa: F401
                    metrics_pb2, model_pb2, objective_functions_pb2, operators_pb2,
                    optimizers_pb2, reader_pb2, trainer_pb2, training_algorithm_pb2,
                    transforms_pb2, weights_pb2)
from .frontend.core import *  # noqa: F401,F403
from .frontend import core as _core
from .frontend.generate import make_iterable, str_list  # noqa: F401
from . import proto  # noqa: F401

__version__ = "0.1.0"

_FEATURES = {"GPU": True, "CUDA": True, "DISTCONV": True, "NVSHMEM": False, "HALF": True,
             "FP16": True, "BF16": True, "ONNX": False, "CNPY": True, "PYTHON": True,
             "TBINF": True, "VISION": True, "CUDNN": False, "DOUBLE": True}


def has_feature(name: str) -> bool:
    """Build features, as ``lbann.has_feature('DISTCONV')`` in the reference."""
    return bool(_FEATURES.get(name.upper(), False))


def lbann_exe():
    return [_sys.executable, "-m", "lbann_b200.driver"]


def run(*args, **kwargs):
    from .launcher import run as _run
    return _run(*args, **kwargs)


def evaluate(*args, **kwargs):
    from .launcher.evaluate import evaluate as _evaluate
    return _evaluate(*args, **kwargs)


def __getattr__(name):
    # lazily loaded sub-packages: lbann.modules, lbann.models, lbann.contrib, lbann.util, ...
    if name == "ops":                      # operator classes (lbann.ops.Clamp, ...): served by the ops package
        import importlib
        return importlib.import_module(f"{__name__}.ops")
    if name in ("modules", "models", "contrib", "util", "launcher", "torch"):
        import importlib
        mod = importlib.import_module(f"{__name__}.{name}")
        globals()[name] = mod
        return mod
    raise AttributeError(f"module '{__name__}' has no attribute '{name}'")
