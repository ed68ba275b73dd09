"""Wrappers of the native kernels (``gemm``, ``conv``, ``nn``, ``optim``, ...).

The front end's ``lbann.ops`` (operator classes such as ``lbann.ops.Clamp``, see
``core/operators.py``) resolves here too, because ``lbann.ops`` and this package share a name:
operator classes are looked up on demand and do not load any kernel wrapper.
"""


def __getattr__(name):
    from ..core import operators as _operators
    if name == "__all__":
        return list(_operators.__all__)
    if name in _operators.__all__:
        return getattr(_operators, name)
    raise AttributeError(f"module '{__name__}' has no attribute '{name}'")
