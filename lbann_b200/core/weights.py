"""Weights and initializer classes."""
from ..frontend import core as _C

for _n in dir(_C):
    _o = getattr(_C, _n)
    if not _n.startswith('_') and (lambda n, o: n == 'Weights' or n == 'Initializer' or n.endswith('Initializer'))(_n, _o):
        globals()[_n] = _o
del _n, _o
