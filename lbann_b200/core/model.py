"""Model and AMP options."""
from ..frontend.core import AmpOptions, Model  # noqa: F401
