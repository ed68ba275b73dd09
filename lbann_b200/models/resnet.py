"""ResNet-18/34/50/101/152 and AlexNet for 2-D image classification.

Same topology and weight naming as the reference's ``lbann.models.ResNet*`` and
``lbann.models.AlexNet`` (python/lbann/models/resnet.py:8-491, alexnet.py:4-85): a 7x7
stride-2 stem with max-pool, four stages of basic or bottleneck residual blocks whose
last batch-norm scale may start at zero, global average pooling and a fully-connected
classifier.
"""
from __future__ import annotations

from ..frontend import core as L
from ..modules.base import Convolution2dModule, FullyConnectedModule, Module


class ConvBNRelu(Module):
    """convolution -> batch normalisation -> optional ReLU."""

    def __init__(self, out_channels, kernel_size, stride, padding, bn_zero_init, bn_statistics_group_size,
                 relu, name):
        super().__init__()
        self.name, self.relu, self.instance = name, relu, 0
        self.conv = Convolution2dModule(out_channels, kernel_size, stride=stride, padding=padding,
                                        bias=False, name=name + "_conv")
        scale0 = 0.0 if bn_zero_init else 1.0
        self.bn_weights = [L.Weights(initializer=L.ConstantInitializer(value=scale0), name=name + "_bn_scale"),
                           L.Weights(initializer=L.ConstantInitializer(value=0.0), name=name + "_bn_bias")]
        self.bn_group = bn_statistics_group_size

    def forward(self, x):
        self.instance += 1
        n = f"{self.name}_instance{self.instance}"
        y = L.BatchNormalization(self.conv(x), weights=self.bn_weights, decay=0.9, epsilon=1e-5,
                                 statistics_group_size=self.bn_group, name=n + "_bn")
        return L.Relu(y, name=n + "_relu") if self.relu else y


class BasicBlock(Module):
    """Two 3x3 convolutions with an identity (or 1x1 projection) shortcut."""

    def __init__(self, in_channels, mid_channels, downsample, zero_init_residual,
                 bn_statistics_group_size, name):
        super().__init__()
        self.name, self.instance = name, 0
        self.out_channels = mid_channels
        stride = 2 if downsample else 1
        self.conv1 = ConvBNRelu(mid_channels, 3, stride, 1, False, bn_statistics_group_size, True,
                                name + "_branch2a")
        self.conv2 = ConvBNRelu(mid_channels, 3, 1, 1, zero_init_residual, bn_statistics_group_size, False,
                                name + "_branch2b")
        self.shortcut = None
        if downsample or in_channels != self.out_channels:
            self.shortcut = ConvBNRelu(self.out_channels, 1, stride, 0, False, bn_statistics_group_size,
                                       False, name + "_branch1")

    def forward(self, x):
        self.instance += 1
        y = self.conv2(self.conv1(x))
        s = self.shortcut(x) if self.shortcut is not None else x
        z = L.Add(y, s, name=f"{self.name}_sum_instance{self.instance}")
        return L.Relu(z, name=f"{self.name}_relu_instance{self.instance}")


class BottleneckBlock(Module):
    """1x1 reduce -> 3x3 -> 1x1 expand (x4) with shortcut."""

    def __init__(self, in_channels, mid_channels, downsample, zero_init_residual,
                 bn_statistics_group_size, name, width=1):
        super().__init__()
        self.name, self.instance = name, 0
        self.out_channels = 4 * mid_channels
        stride = 2 if downsample else 1
        g = bn_statistics_group_size
        inner = mid_channels * width            # wide ResNets widen the inner convolutions only
        self.conv1 = ConvBNRelu(inner, 1, 1, 0, False, g, True, name + "_branch2a")
        self.conv2 = ConvBNRelu(inner, 3, stride, 1, False, g, True, name + "_branch2b")
        self.conv3 = ConvBNRelu(self.out_channels, 1, 1, 0, zero_init_residual, g, False, name + "_branch2c")
        self.shortcut = None
        if downsample or in_channels != self.out_channels:
            self.shortcut = ConvBNRelu(self.out_channels, 1, stride, 0, False, g, False, name + "_branch1")

    def forward(self, x):
        self.instance += 1
        y = self.conv3(self.conv2(self.conv1(x)))
        s = self.shortcut(x) if self.shortcut is not None else x
        z = L.Add(y, s, name=f"{self.name}_sum_instance{self.instance}")
        return L.Relu(z, name=f"{self.name}_relu_instance{self.instance}")


class ResNet(Module):
    global_count = 0

    def __init__(self, block, output_size, layer_sizes, layer_channels, zero_init_residual=True,
                 bn_statistics_group_size=1, name=None, width=1):
        super().__init__()
        ResNet.global_count += 1
        self.name = name or f"resnet_module{ResNet.global_count}"
        self.instance = 0
        g = bn_statistics_group_size
        self.conv1 = ConvBNRelu(layer_channels[0], 7, 2, 3, False, g, True, self.name + "_conv1")
        self.blocks = []
        cin = layer_channels[0]
        for stage, (count, ch) in enumerate(zip(layer_sizes, layer_channels)):
            for i in range(count):
                extra = {"width": width} if width != 1 else {}
                b = block(cin, ch, downsample=(i == 0 and stage > 0), zero_init_residual=zero_init_residual,
                          bn_statistics_group_size=g, name=f"{self.name}_layer{stage + 1}_block{i}", **extra)
                self.blocks.append(b)
                cin = b.out_channels
        self.fc = FullyConnectedModule(output_size, bias=False, name=self.name + "_fc")

    def forward(self, x):
        self.instance += 1
        n = f"{self.name}_instance{self.instance}"
        x = self.conv1(x)
        x = L.Pooling(x, num_dims=2, has_vectors=False, pool_dims_i=3, pool_pads_i=1, pool_strides_i=2,
                      pool_mode="max", name=n + "_pool1")
        for b in self.blocks:
            x = b(x)
        x = L.ChannelwiseMean(x, name=n + "_avgpool")
        return self.fc(x)


def _variant(block, sizes):
    class _R(ResNet):
        def __init__(self, output_size, zero_init_residual=True, bn_statistics_group_size=1, name=None,
                     width=1):
            super().__init__(block, output_size, sizes, tuple(int(c * width) for c in (64, 128, 256, 512)),
                             zero_init_residual=zero_init_residual,
                             bn_statistics_group_size=bn_statistics_group_size, name=name)
    return _R


ResNet18 = _variant(BasicBlock, (2, 2, 2, 2))
ResNet34 = _variant(BasicBlock, (3, 4, 6, 3))
ResNet50 = _variant(BottleneckBlock, (3, 4, 6, 3))
ResNet101 = _variant(BottleneckBlock, (3, 4, 23, 3))
ResNet152 = _variant(BottleneckBlock, (3, 8, 36, 3))
for _n, _c in (("ResNet18", ResNet18), ("ResNet34", ResNet34), ("ResNet50", ResNet50),
               ("ResNet101", ResNet101), ("ResNet152", ResNet152)):
    _c.__name__ = _c.__qualname__ = _n


class AlexNet(Module):
    """Five convolutions (LRN + max-pool after the first two, max-pool after the fifth) and
    three fully-connected layers with dropout (Krizhevsky et al. 2012)."""

    global_count = 0

    def __init__(self, output_size, name=None):
        super().__init__()
        AlexNet.global_count += 1
        self.name = name or f"alexnet_module{AlexNet.global_count}"
        self.instance = 0
        n = self.name
        self.conv1 = Convolution2dModule(96, 11, stride=4, activation=L.Relu, name=n + "_conv1")
        self.conv2 = Convolution2dModule(256, 5, padding=2, activation=L.Relu, name=n + "_conv2")
        self.conv3 = Convolution2dModule(384, 3, padding=1, activation=L.Relu, name=n + "_conv3")
        self.conv4 = Convolution2dModule(384, 3, padding=1, activation=L.Relu, name=n + "_conv4")
        self.conv5 = Convolution2dModule(256, 3, padding=1, activation=L.Relu, name=n + "_conv5")
        self.fc6 = FullyConnectedModule(4096, activation=L.Relu, name=n + "_fc6")
        self.fc7 = FullyConnectedModule(4096, activation=L.Relu, name=n + "_fc7")
        self.fc8 = FullyConnectedModule(output_size, name=n + "_fc8")

    def forward(self, x):
        self.instance += 1
        n = f"{self.name}_instance{self.instance}"

        def pool(x, tag):
            return L.Pooling(x, num_dims=2, has_vectors=False, pool_dims_i=3, pool_pads_i=0,
                             pool_strides_i=2, pool_mode="max", name=f"{n}_pool{tag}")

        def lrn(x, tag):
            return L.LocalResponseNormalization(x, window_width=5, lrn_alpha=0.0001, lrn_beta=0.75,
                                                lrn_k=2, name=f"{n}_norm{tag}")

        x = pool(lrn(self.conv1(x), 1), 1)
        x = pool(lrn(self.conv2(x), 2), 2)
        x = pool(self.conv5(self.conv4(self.conv3(x))), 5)
        x = L.Dropout(self.fc6(x), keep_prob=0.5, name=n + "_drop6")
        x = L.Dropout(self.fc7(x), keep_prob=0.5, name=n + "_drop7")
        return self.fc8(x)


def construct_classifier(net: Module, num_labels: int, num_epochs: int = 1, callbacks=(),
                         l2_weight_decay: float = 0.0):
    """images -> ``net`` -> softmax cross-entropy, top-1 / top-5 accuracy metrics.
    ``l2_weight_decay``: L2 regularisation on the convolution and fully-connected matrices
    (batch-norm parameters and biases excluded), as in the reference's ResNet script
    (applications/vision/resnet.py:96-165)."""
    images = L.Input(data_field="samples", name="images")
    labels = L.Input(data_field="labels", name="labels")
    probs = L.Softmax(net(images), name="probs")
    ce = L.CrossEntropy(probs, labels, name="cross_entropy")
    top1 = L.CategoricalAccuracy(probs, labels, name="top1")
    metrics = [L.Metric(top1, name="top-1 accuracy", unit="%")]
    if num_labels > 5:
        metrics.append(L.Metric(L.TopKCategoricalAccuracy(probs, labels, k=5, name="top5"),
                                name="top-5 accuracy", unit="%"))
    layers = list(L.traverse_layer_graph([images, labels]))
    terms = [ce]
    if l2_weight_decay:
        decayed = set()
        for l in layers:
            if type(l).__name__ in ("Convolution", "FullyConnected") and l.weights:
                decayed.add(l.weights[0])
        if decayed:
            terms.append(L.L2WeightRegularization(weights=list(decayed), scale=l2_weight_decay))
    return L.Model(num_epochs, layers=layers, objective_function=L.ObjectiveFunction(terms),
                   metrics=metrics, callbacks=list(callbacks))
