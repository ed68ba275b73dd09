"""Callbacks: hook interface, registry and the built-in set."""
from .base import CALLBACK_REGISTRY, ExecCallback, build_callback, register  # noqa: F401
from . import standard  # noqa: F401
from . import io_misc  # noqa: F401
