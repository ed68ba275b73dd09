"""Compatibility name: ``import lbann`` resolves to ``lbann_b200``.

Scripts written for the reference front end (``import lbann``, ``lbann.modules``,
``lbann.models``, ``lbann.contrib.args``, ``lbann.util.data`` ...) run unchanged.
"""
import importlib as _importlib
import sys as _sys

import lbann_b200 as _impl

_this = _sys.modules[__name__]
for _k in dir(_impl):
    if not _k.startswith("__"):
        setattr(_this, _k, getattr(_impl, _k))
__version__ = _impl.__version__


class _AliasFinder:
    """Maps ``lbann.<sub>`` imports onto ``lbann_b200.<sub>``."""

    @staticmethod
    def find_spec(name, path=None, target=None):
        if not name.startswith("lbann."):
            return None
        real = "lbann_b200." + name[len("lbann."):]
        try:
            mod = _importlib.import_module(real)
        except ImportError:
            return None
        _sys.modules[name] = mod
        from importlib.machinery import ModuleSpec

        class _Loader:
            @staticmethod
            def create_module(spec):
                return mod

            @staticmethod
            def exec_module(module):
                pass
        return ModuleSpec(name, _Loader())


_sys.meta_path.insert(0, _AliasFinder)


def __getattr__(name):
    return getattr(_impl, name)
