"""Experimental models (python/lbann/contrib/models)."""
from .wide_resnet import WideResNet50_2  # noqa: F401
