"""``lbann.models``: model zoo (LeNet, AlexNet, ResNet, CosmoFlow, U-Net3D, Transformer / GPT, RoBERTa,
sub-graph Transformer)."""
from .lenet import LeNet  # noqa: F401
from .cosmoflow import CosmoFlow, construct_cosmoflow_model  # noqa: F401
from .resnet import (AlexNet, ResNet, ResNet18, ResNet34, ResNet50, ResNet101, ResNet152,  # noqa: F401
                     construct_classifier)
from .transformer import (GPT, LayerNorm, Transformer, TransformerDecoderLayer,  # noqa: F401
                          TransformerEncoderLayer, causal_mask, construct_gpt_model)
from .unet3d import UNet3D, construct_unet3d_model  # noqa: F401
from .roberta import RoBERTa, RobertaConfig  # noqa: F401
from . import subgraph  # noqa: F401
