"""Reusable layer patterns with shared weights (``lbann.modules``).

A module is a callable that adds layers to the graph every time it is applied; all
applications share the module's weights.  Names follow the reference so that weights
names in checkpoints agree: ``<name>_matrix`` / ``<name>_bias`` for fully-connected
modules, ``<name>_kernel`` / ``<name>_bias`` for convolutions, layers
``<name>_instance<k>[_fc|_conv|_deconv|_activation]`` (python/lbann/modules/base.py:38-370).
"""
from __future__ import annotations

from ..frontend import core as L
from ..frontend.generate import make_iterable, str_list


class Module:
    """Base class: subclasses implement ``forward(*inputs)``."""

    def __init__(self):
        pass

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)


def _make_weights(weights, count, names, initializers):
    ws = list(make_iterable(weights)) if weights is not None else []
    if len(ws) > count:
        raise ValueError(f"at most {count} weights expected, got {len(ws)}")
    out = []
    for i in range(count):
        if i < len(ws) and ws[i] is not None:
            w = ws[i]
        else:
            w = L.Weights(initializer=initializers[i]())
        if w.name is None or w.name.startswith("weights"):
            w.name = names[i]
        out.append(w)
    return out


class FullyConnectedModule(Module):
    global_count = 0

    def __init__(self, size, bias=True, transpose=False, weights=None, activation=None, name=None,
                 data_layout="data_parallel", parallel_strategy=None):
        super().__init__()
        FullyConnectedModule.global_count += 1
        self.instance = 0
        self.size, self.bias, self.transpose = size, bias, transpose
        self.name = name or f"fcmodule{FullyConnectedModule.global_count}"
        self.data_layout = data_layout
        self.parallel_strategy = parallel_strategy or {}
        self.weights = _make_weights(weights, 2 if bias else 1,
                                     [self.name + "_matrix", self.name + "_bias"],
                                     [L.HeNormalInitializer, lambda: L.ConstantInitializer(value=0.0)])
        self.activation = None
        if activation is not None:
            self.activation = activation if isinstance(activation, type) or callable(activation) else None
            if self.activation is None:
                raise ValueError("activation must be a layer class or callable")

    def forward(self, x):
        self.instance += 1
        name = f"{self.name}_instance{self.instance}"
        y = L.FullyConnected(x, weights=self.weights, name=(name + "_fc" if self.activation else name),
                             data_layout=self.data_layout, num_neurons=self.size, has_bias=self.bias,
                             transpose=self.transpose, parallel_strategy=self.parallel_strategy)
        if self.activation:
            return self.activation(y, name=name + "_activation", data_layout=self.data_layout,
                                   parallel_strategy=self.parallel_strategy)
        return y


class ChannelwiseFullyConnectedModule(Module):
    global_count = 0

    def __init__(self, size, bias=True, transpose=False, weights=None, activation=None, name=None,
                 parallel_strategy=None, data_layout=None):
        super().__init__()
        ChannelwiseFullyConnectedModule.global_count += 1
        self.instance = 0
        self.size = list(make_iterable(size))
        self.bias, self.transpose = bias, transpose
        self.name = name or f"channelwisefc{ChannelwiseFullyConnectedModule.global_count}"
        self.parallel_strategy = parallel_strategy or {}
        self.data_layout = data_layout
        self.weights = _make_weights(weights, 2 if bias else 1,
                                     [self.name + "_matrix", self.name + "_bias"],
                                     [L.HeNormalInitializer, lambda: L.ConstantInitializer(value=0.0)])
        self.activation = activation

    def forward(self, x):
        self.instance += 1
        name = f"{self.name}_instance{self.instance}"
        kw = {"data_layout": self.data_layout} if self.data_layout else {}
        y = L.ChannelwiseFullyConnected(x, weights=self.weights,
                                        name=(name + "_fc" if self.activation else name),
                                        output_channel_dims=self.size, bias=self.bias,
                                        transpose=self.transpose,
                                        parallel_strategy=self.parallel_strategy, **kw)
        if self.activation:
            return self.activation(y, name=name + "_activation",
                                   parallel_strategy=self.parallel_strategy)
        return y


class ConvolutionModule(Module):
    global_count = 0

    def __init__(self, num_dims, out_channels, kernel_size, stride=1, padding=0, dilation=1,
                 groups=1, bias=True, weights=None, activation=None, name=None, transpose=False,
                 parallel_strategy=None):
        super().__init__()
        ConvolutionModule.global_count += 1
        self.instance = 0
        self.num_dims, self.out_channels = num_dims, out_channels
        self.kernel_size, self.stride = kernel_size, stride
        self.padding, self.dilation, self.groups = padding, dilation, groups
        self.bias, self.transpose = bias, transpose
        self.name = name or f"convmodule{ConvolutionModule.global_count}"
        self.parallel_strategy = parallel_strategy or {}
        self.weights = _make_weights(weights, 2 if bias else 1,
                                     [self.name + "_kernel", self.name + "_bias"],
                                     [L.HeNormalInitializer, lambda: L.ConstantInitializer(value=0.0)])
        self.activation = activation

    def _vec(self, v):
        v = list(make_iterable(v))
        return v * self.num_dims if len(v) == 1 else v

    def forward(self, x):
        self.instance += 1
        name = f"{self.name}_instance{self.instance}"
        cls = L.Deconvolution if self.transpose else L.Convolution
        suffix = "_deconv" if self.transpose else "_conv"
        y = cls(x, weights=self.weights, name=(name + suffix if self.activation else name),
                num_dims=self.num_dims, out_channels=self.out_channels,
                kernel_size=self._vec(self.kernel_size), stride=self._vec(self.stride),
                padding=self._vec(self.padding), dilation=self._vec(self.dilation),
                groups=self.groups, has_bias=self.bias, parallel_strategy=self.parallel_strategy)
        if self.activation:
            return self.activation(y, name=name + "_activation",
                                   parallel_strategy=self.parallel_strategy)
        return y


class Convolution2dModule(ConvolutionModule):
    def __init__(self, *args, **kwargs):
        super().__init__(2, *args, **kwargs)


class Convolution3dModule(ConvolutionModule):
    def __init__(self, *args, **kwargs):
        super().__init__(3, *args, **kwargs)
