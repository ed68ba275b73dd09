"""Wide ResNet-50-2 (Zagoruyko & Komodakis 2016; python/lbann/contrib/models/wide_resnet.py):
ResNet-50 whose bottleneck 3x3 convolutions are twice as wide, output widths unchanged."""
from __future__ import annotations

from ...models.resnet import BottleneckBlock, ResNet


class WideResNet50_2(ResNet):
    global_count = 0

    def __init__(self, output_size, zero_init_residual=True, bn_statistics_group_size=1, name=None):
        WideResNet50_2.global_count += 1
        name = name or f"wide_resnet50_module{WideResNet50_2.global_count}"
        super().__init__(BottleneckBlock, output_size, (3, 4, 6, 3), (64, 128, 256, 512),
                         zero_init_residual, bn_statistics_group_size, name, width=2)
