"""Mixed-precision helpers (``lbann.util.amp``, python/lbann/util/amp.py:38-197): give every
learnable layer explicit weights objects, keep master weights in fp32 and run the layers
in a 16-bit datatype with loss scaling."""
from __future__ import annotations

from ..frontend import core as L

_WEIGHTED = {"FullyConnected": 2, "ChannelwiseFullyConnected": 2, "Convolution": 2, "Deconvolution": 2,
             "BatchNormalization": 4, "LayerNorm": 2, "Embedding": 1, "ChannelwiseScaleBias": 1,
             "EntrywiseScaleBias": 1, "InstanceNorm": 0, "GRU": 4}


def num_weights_by_bias(layer, bias_field: str = "has_bias") -> int:
    """2 with a bias term, 1 without."""
    v = getattr(layer, bias_field, None)
    return 2 if (v is None or bool(v)) else 1


def add_weights(model) -> None:
    """Attach explicit ``lbann.Weights`` objects to layers that would create theirs
    implicitly, so that their datatype can be pinned to fp32."""
    for l in model.layers:
        n = _WEIGHTED.get(type(l).__name__)
        if n is None:
            continue
        if type(l).__name__ in ("FullyConnected", "Convolution", "Deconvolution"):
            n = num_weights_by_bias(l)
        elif type(l).__name__ == "ChannelwiseFullyConnected":
            n = num_weights_by_bias(l, "bias")
        while len(l.weights) < n:
            l.weights.append(L.Weights(datatype=L.DataType.FLOAT))


def get_widest_datatype(datatypes):
    order = [L.DataType.FP16, L.DataType.FLOAT, L.DataType.DOUBLE]
    return max(datatypes, key=lambda d: order.index(d) if d in order else 1)


def set_layer_datatypes(model, datatype=None) -> None:
    dt = datatype if datatype is not None else L.DataType.FP16
    for l in model.layers:
        if l.datatype is None:
            l.datatype = dt


def enable_amp(model, init_scale=None, growth_factor=None, backoff_factor=None, growth_interval=None,
               datatype=None) -> None:
    """16-bit layers, fp32 master weights, dynamic loss scaling."""
    add_weights(model)
    set_layer_datatypes(model, datatype)
    model.amp = L.AmpOptions(enabled=True, init_scale=init_scale, growth_factor=growth_factor,
                             backoff_factor=backoff_factor, growth_interval=growth_interval)
