"""Defaults for the machines of this computing centre (python/lbann/contrib/nersc)."""
from . import launcher, paths, systems  # noqa: F401
