"""Defaults for the machines of this computing centre (python/lbann/contrib/riken)."""
from . import launcher, paths, systems  # noqa: F401
