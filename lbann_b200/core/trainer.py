"""Trainer."""
from ..frontend.core import Trainer  # noqa: F401
