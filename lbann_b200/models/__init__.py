"""``lbann.models``: model zoo (LeNet, AlexNet, ResNet, CosmoFlow, U-Net3D, Transformer / GPT)."""
from .lenet import LeNet  # noqa: F401
from .cosmoflow import CosmoFlow, construct_cosmoflow_model  # noqa: F401
