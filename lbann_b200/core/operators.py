"""Operator classes (``lbann.ops``): the entry-wise operators that an ``OperatorLayer`` chains,
one class per operator message of the schema, e.g.

    lbann.OperatorLayer(x, ops=[lbann.ops.Clamp(min=0.0, max=1.0)])

(python/lbann/core/operators.py generates the same classes from operators.proto)."""
from ..frontend.core import Operator, operator_classes as _classes

globals().update(_classes)
__all__ = ["Operator"] + sorted(_classes)
