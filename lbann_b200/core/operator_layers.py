"""Layer classes that wrap a single operator (``lbann.Add``, ``lbann.Relu`` ...)."""
from ..frontend import core as _C

for _n in dir(_C):
    _o = getattr(_C, _n)
    if isinstance(_o, type) and issubclass(_o, _C.Layer) and getattr(_o, '_operator', None) is not None:
        globals()[_n] = _o
del _n, _o
