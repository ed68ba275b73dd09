"""Experimental modules (python/lbann/contrib/modules)."""
from .fftshift import FFTShift  # noqa: F401
from .radial_profile import RadialProfile  # noqa: F401
from . import objective_functions  # noqa: F401
