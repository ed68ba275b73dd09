"""3-D U-Net for volumetric segmentation with distconv spatial parallelism.

Four down / up levels of (conv3d 3x3x3 + batch norm + ReLU) x 2, max-pool 2 on the way
down, transposed convolution (kernel 2, stride 2) on the way up with skip concatenation,
a 1x1x1 classifier and per-voxel softmax cross-entropy - the architecture of the
reference's ``applications/vision/unet3d.py`` (lines 29-260).  Every convolution,
normalisation, activation, pooling and loss layer carries the given
``parallel_strategy`` so that the executor partitions them spatially.
"""
from __future__ import annotations

from ..frontend import core as L
from ..modules.base import Convolution3dModule, ConvolutionModule, Module


class _ConvBNRelu3d(Module):
    def __init__(self, channels, name, ps, bn_group):
        super().__init__()
        self.name, self.ps, self.bn_group, self.instance = name, ps, bn_group, 0
        self.conv = Convolution3dModule(channels, 3, stride=1, padding=1, bias=False, name=name + "_conv",
                                        parallel_strategy=ps)
        self.bn_weights = [L.Weights(initializer=L.ConstantInitializer(value=1.0), name=name + "_bn_scale"),
                           L.Weights(initializer=L.ConstantInitializer(value=0.0), name=name + "_bn_bias")]

    def forward(self, x):
        self.instance += 1
        n = f"{self.name}_instance{self.instance}"
        y = L.BatchNormalization(self.conv(x), weights=self.bn_weights, decay=0.9, epsilon=1e-5,
                                 statistics_group_size=self.bn_group, name=n + "_bn",
                                 parallel_strategy=self.ps)
        return L.Relu(y, name=n + "_relu", parallel_strategy=self.ps)


class UNet3D(Module):
    global_count = 0

    def __init__(self, num_classes=3, base_channels=32, levels=4, parallel_strategy=None,
                 bn_statistics_group_size=0, name=None):
        super().__init__()
        UNet3D.global_count += 1
        self.name = name or f"unet3d_module{UNet3D.global_count}"
        self.ps = parallel_strategy or {}
        self.levels, self.num_classes = levels, num_classes
        g = bn_statistics_group_size
        ch = [base_channels * 2 ** i for i in range(levels + 1)]
        self.down = [[_ConvBNRelu3d(ch[i], f"{self.name}_down{i}_a", self.ps, g),
                      _ConvBNRelu3d(ch[i] * 2 if i < levels else ch[i], f"{self.name}_down{i}_b", self.ps, g)]
                     for i in range(levels + 1)]
        self.up_deconv, self.up = [], []
        for i in reversed(range(levels)):
            self.up_deconv.append(ConvolutionModule(3, ch[i + 1], 2, stride=2, padding=0, bias=False,
                                                    transpose=True, name=f"{self.name}_up{i}_deconv",
                                                    parallel_strategy=self.ps))
            self.up.append([_ConvBNRelu3d(ch[i + 1], f"{self.name}_up{i}_a", self.ps, g),
                            _ConvBNRelu3d(ch[i + 1], f"{self.name}_up{i}_b", self.ps, g)])
        self.classifier = Convolution3dModule(num_classes, 1, stride=1, padding=0, bias=True,
                                              name=f"{self.name}_classifier", parallel_strategy=self.ps)

    def forward(self, x):
        skips = []
        for i, (a, b) in enumerate(self.down):
            x = b(a(x))
            if i < self.levels:
                skips.append(x)
                x = L.Pooling(x, num_dims=3, has_vectors=False, pool_dims_i=2, pool_pads_i=0,
                              pool_strides_i=2, pool_mode="max", name=f"{self.name}_pool{i}",
                              parallel_strategy=self.ps)
        for j, (deconv, (a, b)) in enumerate(zip(self.up_deconv, self.up)):
            x = deconv(x)
            x = L.Concatenation([skips[-1 - j], x], axis=0, name=f"{self.name}_cat{j}",
                                parallel_strategy=self.ps)
            x = b(a(x))
        return self.classifier(x)


def construct_unet3d_model(num_classes=3, base_channels=32, levels=4, num_epochs=1,
                           parallel_strategy=None, bn_statistics_group_size=0, callbacks=(),
                           label_field="responses"):
    """volume ``[1, D, H, W]`` + per-voxel integer labels ``[D, H, W]`` (data field
    ``label_field``) -> summed per-voxel cross-entropy."""
    ps = parallel_strategy or {}
    vol = L.Input(data_field="samples", name="volume")
    lab = L.Input(data_field=label_field, name="voxel_labels")
    net = UNet3D(num_classes, base_channels, levels, ps, bn_statistics_group_size)
    logits = net(vol)
    probs = L.Softmax(logits, softmax_mode="channel", name="voxel_probs", parallel_strategy=ps)
    ce = L.CrossEntropy(probs, lab, use_labels=True, name="voxel_ce", parallel_strategy=ps)
    layers = list(L.traverse_layer_graph([vol, lab]))
    return L.Model(num_epochs, layers=layers, objective_function=L.ObjectiveFunction([ce]),
                   metrics=[L.Metric(ce, name="cross entropy")], callbacks=list(callbacks))
