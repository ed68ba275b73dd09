"""Objective function and its terms."""
from ..frontend.core import L2WeightRegularization, LayerTerm, ObjectiveFunction  # noqa: F401
