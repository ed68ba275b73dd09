"""Metric."""
from ..frontend.core import Metric  # noqa: F401
