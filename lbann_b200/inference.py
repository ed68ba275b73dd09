"""Embedding the framework in another application: initialise, load a trained model, infer.

The reference ships a small C++ client (core-driver/main.cpp:67-137) that calls
``initialize_lbann(MPI_Comm)``, ``load_inference_model`` (src/utils/lbann_library.cpp:55-70: a
model saved by the checkpoint / save-model callbacks, rebuilt with a given mini-batch size and
input / output dimensions) and runs the batch inference algorithm on matrices it owns.  This
module is that surface for Python callers; ``python -m lbann_b200.inference`` is the example
client.
"""
from __future__ import annotations

import glob
import os
from typing import Optional, Sequence

import numpy as np
import torch

from .driver import load_prototext
from .utils import options as opts


def initialize_lbann(argv: Optional[Sequence[str]] = None):
    """Parse framework options (``--disable_cuda`` ...) and return the option store; the
    communicator is created by the trainer, one process per GPU."""
    o = opts.reset()
    o.parse(list(argv or []))
    return o


def finalize_lbann(handle=None) -> None:
    if handle is not None:
        handle.trainer.shutdown()


class InferenceModel:
    def __init__(self, trainer, model, mini_batch_size: int):
        self.trainer, self.model, self.mini_batch_size = trainer, model, mini_batch_size

    def _inputs(self, field, xb):
        """The given field plus zeros for the model's other inputs (labels / responses feed
        the loss layers, which inference does not read)."""
        feed = {field: xb}
        dc = self.trainer.data_coordinator
        for l in self.model.layers:
            if l.type == "input" and l.field not in feed:
                feed[l.field] = torch.zeros((xb.shape[0],) + tuple(dc.dims(l.field)), device=xb.device)
        return feed

    def infer(self, samples, field: str = "samples", output_layer: Optional[str] = None,
              labels: bool = False):
        """``samples``: ``[n, ...]`` array or tensor.  Returns the outputs of ``output_layer``
        (default: the last layer) as a NumPy array, or arg-max labels with ``labels=True``."""
        x = torch.as_tensor(np.asarray(samples, dtype=np.float32)) if not torch.is_tensor(samples) else samples
        x = x.reshape(x.shape[0], -1)
        if labels:
            return self.infer(x, field, output_layer).reshape(x.shape[0], -1).argmax(1)
        layer = output_layer or self.model.layers[-1].name
        outs = []
        with torch.no_grad():
            for i in range(0, x.shape[0], self.mini_batch_size):
                xb = x[i:i + self.mini_batch_size].to(self.model.device)
                self.model.forward_prop(self._inputs(field, xb), "prediction")
                outs.append(self.model.acts[layer][0].float().cpu())
        return torch.cat(outs).numpy() if outs else np.zeros((0,), dtype=np.float32)


def load_inference_model(directory: str, mini_batch_size: int, input_dims,
                         prototext: Optional[str] = None) -> InferenceModel:
    """``directory``: what the save-model / checkpoint callbacks wrote (weights, and the
    experiment prototext unless ``prototext`` names it).  ``input_dims``: dimensions of one
    sample of the ``samples`` field, or a dict field -> dimensions.  The model is rebuilt for
    ``mini_batch_size`` and its weights are loaded; no optimizer state is created."""
    from .data.readers import ArrayReader
    from .exec.trainer import ExecTrainer
    from .io import checkpoint
    proto_path = prototext
    if proto_path is None:
        cands = sorted(glob.glob(os.path.join(directory, "**", "*.prototext"), recursive=True))
        if not cands:
            raise FileNotFoundError(f"no model prototext under {directory}")
        proto_path = cands[0]
    msg = load_prototext(proto_path)
    msg.trainer.mini_batch_size = int(mini_batch_size)
    msg.optimizer.Clear()
    msg.optimizer.no_optimizer.SetInParent()
    for w in msg.model.weights:
        w.ClearField("optimizer")
    dims = input_dims if isinstance(input_dims, dict) else {"samples": tuple(input_dims)}
    arrays = {f: np.zeros((1,) + tuple(d), dtype=np.float32) for f, d in dims.items()}
    trainer = ExecTrainer(msg, readers={"test": ArrayReader(arrays, role="test")})
    model = trainer.build_model(msg.model)
    saved = sorted(glob.glob(os.path.join(directory, "**", "model.bin"), recursive=True),
                   key=os.path.getmtime)
    if not saved:
        raise FileNotFoundError(f"no saved model (model.bin) under {directory}")
    checkpoint.load_model(model, saved[-1], strict=False)
    return InferenceModel(trainer, model, int(mini_batch_size))


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="load a saved model and run it on random inputs")
    ap.add_argument("directory")
    ap.add_argument("--prototext")
    ap.add_argument("--mini-batch-size", type=int, default=8)
    ap.add_argument("--samples", type=int, default=16)
    ap.add_argument("--input-dims", type=int, nargs="+", required=True, help="dimensions of one sample")
    a, rest = ap.parse_known_args(argv)
    initialize_lbann(rest)
    h = load_inference_model(a.directory, a.mini_batch_size, a.input_dims, a.prototext)
    out = h.infer(np.random.randn(a.samples, *a.input_dims).astype(np.float32), labels=True)
    print("predicted labels:", out.tolist())
    finalize_lbann(h)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
