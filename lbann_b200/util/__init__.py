"""``lbann.util``: small helpers shared by the front end and applications."""
from ..frontend.generate import make_iterable, str_list  # noqa: F401
from . import amp, data  # noqa: F401
