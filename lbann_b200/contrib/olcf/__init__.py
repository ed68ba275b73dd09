"""Defaults for the machines of this computing centre (python/lbann/contrib/olcf)."""
from . import launcher, paths, systems  # noqa: F401
