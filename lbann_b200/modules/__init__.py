"""``lbann.modules``: reusable layer patterns with shared weights."""
from .base import (ChannelwiseFullyConnectedModule, Convolution2dModule, Convolution3dModule,  # noqa: F401
                   ConvolutionModule, FullyConnectedModule, Module)
