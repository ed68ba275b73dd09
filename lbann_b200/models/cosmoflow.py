"""CosmoFlow 3-D CNN (applications/physics/cosmology/cosmoflow/
cosmoflow_network_architectures.py:8-252, cosmoflow_model.py:5-90 of the reference).

``num_conv = log2(width) - 2`` blocks of conv 3x3x3 -> leaky ReLU(0.3) -> pool 2, then
fully-connected 2048 / 256 / output (MLPerf variant: 128 / 64 / output, max-pool, wider
channels), mean-squared-error loss.  Convolutions carry no bias when a spatial
``parallel_strategy`` is given (cosmoflow_model.py:52).
"""
from __future__ import annotations

import math
from functools import partial

from ..frontend import core as L
from ..modules import Convolution3dModule, FullyConnectedModule, Module


class CosmoFlow(Module):
    global_count = 0

    def __init__(self, input_width, output_size, name=None, channels=None, pool_mode="average",
                 fc_sizes=(2048, 256), use_bn=False, bn_statistics_group_size=1,
                 dropout_keep_prob=1.0, parallel_strategy=None, conv_bias=None, mlperf=False):
        super().__init__()
        CosmoFlow.global_count += 1
        self.name = name or f"cosmoflow_module{CosmoFlow.global_count}"
        n_conv = int(math.log2(input_width)) - 2
        if channels is None:
            base, cap = (32, 512) if mlperf else (16, 256)
            channels = [min(base * 2 ** i, cap) for i in range(n_conv)]
        if mlperf:
            fc_sizes, pool_mode = (128, 64), "max"
        self.channels = list(channels)
        self.pool_mode = pool_mode
        self.use_bn = use_bn
        self.bn_group = bn_statistics_group_size
        self.keep = dropout_keep_prob
        self.ps = parallel_strategy or {}
        bias = (not self.ps) if conv_bias is None else conv_bias
        self.convs = [Convolution3dModule(c, 3, stride=1, padding=1, bias=bias and not use_bn,
                                          name=f"{self.name}_conv{i + 1}", parallel_strategy=self.ps)
                      for i, c in enumerate(self.channels)]
        sizes = list(fc_sizes) + [output_size]
        self.fcs = []
        for i, s in enumerate(sizes):
            init = L.HeNormalInitializer() if i < len(sizes) - 1 else L.ConstantInitializer(value=0.0)
            self.fcs.append(FullyConnectedModule(
                s, name=f"{self.name}_fc{i + 1}",
                weights=[L.Weights(initializer=init), L.Weights(initializer=L.ConstantInitializer(value=0.0))]))

    def forward(self, x):
        act = partial(L.LeakyRelu, negative_slope=0.3)
        for i, conv in enumerate(self.convs):
            x = conv(x)
            if self.use_bn:
                x = L.BatchNormalization(x, statistics_group_size=self.bn_group, epsilon=1e-5,
                                         decay=0.9, name=f"{self.name}_bn{i + 1}",
                                         parallel_strategy=self.ps)
            x = act(x, name=f"{self.name}_act{i + 1}", parallel_strategy=self.ps)
            x = L.Pooling(x, num_dims=3, has_vectors=False, pool_dims_i=2, pool_pads_i=0,
                          pool_strides_i=2, pool_mode=self.pool_mode, name=f"{self.name}_pool{i + 1}",
                          parallel_strategy=self.ps)
        for i, fc in enumerate(self.fcs):
            x = fc(x)
            if i < len(self.fcs) - 1:
                x = act(x, name=f"{self.name}_fc_act{i + 1}")
                if self.keep < 1.0:
                    x = L.Dropout(x, keep_prob=self.keep)
        return x


def construct_cosmoflow_model(input_width=128, in_channels=4, num_outputs=4, num_epochs=1,
                              channels=(32, 64, 128, 256, 256), pool_mode="max",
                              parallel_strategy=None, use_bn=False, callbacks=(), **kw):
    """Model for the benchmark configuration: input ``in_channels`` x width^3 volumes in the
    ``samples`` field, ``num_outputs`` regression targets in ``responses``, MSE objective."""
    images = L.Input(data_field="samples", name="input_volume")
    targets = L.Input(data_field="responses", name="input_targets")
    net = CosmoFlow(input_width, num_outputs, channels=list(channels), pool_mode=pool_mode,
                    use_bn=use_bn, parallel_strategy=parallel_strategy, **kw)
    preds = net(images)
    mse = L.MeanSquaredError(preds, targets, name="mse")
    return L.Model(num_epochs, layers=[images, targets], objective_function=[L.LayerTerm(mse)],
                   metrics=[L.Metric(mse, name="MSE")], callbacks=list(callbacks),
                   name="cosmoflow")


def synthetic_reader(num_samples, input_width=128, in_channels=4, num_outputs=4, pool=0):
    from ..proto import lbann_pb2 as pb
    rd = pb.DataReader()
    r = rd.reader.add()
    r.name, r.role, r.shuffle = "synthetic", "train", False
    r.num_samples = num_samples
    r.synth_dimensions = f"{in_channels} {input_width} {input_width} {input_width}"
    r.synth_response_dimensions = str(num_outputs)
    r.synth_distribution = "samples:lognormal responses:uniform_pm1"
    r.fraction_of_data_to_use = 1.0
    if pool:
        r.synth_pool_size = pool
    return rd
