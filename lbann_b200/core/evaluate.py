"""``lbann.evaluate``."""
from ..launcher.evaluate import evaluate  # noqa: F401
