"""Metrics that are not read from a layer (src/metrics/{executable,python}_metric.cpp)."""
from __future__ import annotations

import importlib
import subprocess
import sys


class ExternalMetric:
    layer_name = None

    def __init__(self, name, unit=""):
        self.name, self.unit = name, unit

    def evaluate(self, model, mode) -> float:
        raise NotImplementedError


class ExecutableMetric(ExternalMetric):
    """Runs ``<filename> <other_args> <experiment dir>`` and parses the last number printed."""

    def __init__(self, msg):
        super().__init__(msg.name)
        self.filename, self.args = msg.filename, msg.other_args

    def evaluate(self, model, mode):
        out = subprocess.run([self.filename] + self.args.split(), capture_output=True, text=True,
                             check=True).stdout.split()
        return float(out[-1])


class PythonMetric(ExternalMetric):
    """Calls ``module.function(experiment_dir)`` in this process."""

    def __init__(self, msg):
        super().__init__(msg.name)
        if msg.module_dir and msg.module_dir not in sys.path:
            sys.path.insert(0, msg.module_dir)
        self.fn = getattr(importlib.import_module(msg.module), msg.function or "evaluate")

    def evaluate(self, model, mode):
        import os
        return float(self.fn(os.getcwd()))


def make_external_metric(which, msg):
    return ExecutableMetric(msg) if which == "executable_metric" else PythonMetric(msg)
