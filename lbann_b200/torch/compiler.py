"""``lbann.torch.compile``: trace a PyTorch module with ``torch.fx`` and lower it to front-end
layers (python/lbann/torch/compiler.py).  The pieces: ``opaque`` (tracing, with registered
module classes kept whole), ``lowering`` (graph walk), ``converters`` (per-module / per-function
rules), ``helpers``."""
from .converters import register_function, register_module  # noqa: F401
from .lowering import compile  # noqa: F401
