"""``lbann.torch``: turn a PyTorch module into an LBANN layer graph.

``compile(module, x=example)`` traces the module with ``torch.fx`` and lowers every node
it knows to front-end layers, copying parameters into ``lbann.Weights`` when
``with_weights=True`` (python/lbann/torch/compiler.py:54-199, lowering.py:44-446,
converters.py:64-193).  Unknown modules / functions raise with the node's name;
``register_module`` / ``register_function`` add converters.
"""
from .compiler import compile, register_function, register_module  # noqa: F401
from .opaque import register_opaque  # noqa: F401
