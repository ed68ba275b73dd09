"""LeNet-5 (python/lbann/models/lenet.py, applications/vision/lenet.py:22-68)."""
from __future__ import annotations

from ..frontend import core as L
from ..modules import Convolution2dModule, FullyConnectedModule, Module


class LeNet(Module):
    global_count = 0

    def __init__(self, output_size, name=None):
        super().__init__()
        LeNet.global_count += 1
        self.name = name or f"lenet_module{LeNet.global_count}"
        self.conv1 = Convolution2dModule(6, 5, activation=L.Relu, name=self.name + "_conv1")
        self.conv2 = Convolution2dModule(16, 5, activation=L.Relu, name=self.name + "_conv2")
        self.fc1 = FullyConnectedModule(120, activation=L.Relu, name=self.name + "_fc1")
        self.fc2 = FullyConnectedModule(84, activation=L.Relu, name=self.name + "_fc2")
        self.fc3 = FullyConnectedModule(output_size, name=self.name + "_fc3")

    def forward(self, x):
        x = self.conv1(x)
        x = L.Pooling(x, num_dims=2, pool_dims_i=2, pool_pads_i=0, pool_strides_i=2, pool_mode="max")
        x = self.conv2(x)
        x = L.Pooling(x, num_dims=2, pool_dims_i=2, pool_pads_i=0, pool_strides_i=2, pool_mode="max")
        return self.fc3(self.fc2(self.fc1(x)))
