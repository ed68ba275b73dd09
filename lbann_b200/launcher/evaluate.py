"""``lbann.evaluate``: run a model (or a bare layer graph) once on NumPy inputs and return
the forward outputs as NumPy arrays.

Same contract as the reference's helper (python/lbann/core/evaluate.py:40-150), which
writes the inputs to disk, launches the executable with dump callbacks and reads the
dumps back; here the model is built and executed in-process, so nothing touches disk.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..frontend import core as L


def evaluate(model, inputs: np.ndarray, outputs: Optional[Sequence[str]] = None,
             extra_callbacks: Optional[List] = None, training: bool = False, **kwargs):
    """``model``: an ``lbann.Model``, a layer or a list of layers.  ``inputs``:
    ``[samples, ...]`` array mapped to the ``samples`` data field.  ``outputs``: layer
    names to return (default: every layer without children).  Returns one array, or a
    tuple of arrays when several outputs are requested."""
    from ..data.readers import ArrayReader
    from ..exec.trainer import ExecTrainer
    from ..proto import serialize

    if isinstance(model, L.Layer):
        model = [model]
    if isinstance(model, (list, tuple, set)):
        model = L.Model(0, layers=list(L.traverse_layer_graph(list(model))))
    if not outputs:
        outputs = [l.name for l in model.layers if not l.children]
    outputs = list(outputs)
    if extra_callbacks:
        model.callbacks = list(model.callbacks) + list(extra_callbacks)

    x = np.ascontiguousarray(inputs, dtype=np.float32)
    n = x.shape[0]
    exp = serialize.build_experiment(
        trainer=L.Trainer(mini_batch_size=n), model=model, data_reader=None,
        optimizer=kwargs.get("optimizer") or L.NoOptimizer())
    role = "train" if training else "test"
    tr = ExecTrainer(exp, readers={role: ArrayReader({"samples": x}, role=role)})
    try:
        m = tr.build_model(exp.model)
        mode = "training" if training else "testing"
        dc = tr.data_coordinator
        dc.start_epoch(mode)
        batch = dc.next_batch(mode)
        with torch.no_grad():
            m.forward_prop(batch.tensors, mode, batch.global_size, 0)
        res = []
        for name in outputs:
            if name not in m.acts:
                raise KeyError(f"evaluate: the model has no layer named '{name}'")
            res.append(m.acts[name][0].detach().float().cpu().numpy())
    finally:
        tr.shutdown()
    return res[0] if len(res) == 1 else tuple(res)
