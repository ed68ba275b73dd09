"""Helpers of the lowering: parameters as ``lbann.Weights`` with their values, the context
that carries sample shapes from ``torch.fx`` shape propagation (python/lbann/torch/helpers.py)."""
from __future__ import annotations

import operator
from typing import Callable, Dict, List

import numpy as np
import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

from ..frontend import core as L


def _weights(t: torch.Tensor, name: str, trainable: bool = True):
    vals = t.detach().float().cpu().numpy()
    return L.Weights(initializer=L.ValueInitializer(values=vals.reshape(-1).tolist()), name=name,
                     optimizer=None if trainable else L.NoOptimizer())


class _Ctx:
    def __init__(self, with_weights):
        self.with_weights = with_weights
        self.shapes = {}
