"""AlexNet (python/lbann/models/alexnet.py); the module is defined beside the residual
networks, whose building blocks it shares."""
from .resnet import AlexNet  # noqa: F401
