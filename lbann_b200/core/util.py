"""Small helpers of the front end."""
from ..frontend.generate import make_iterable, str_list  # noqa: F401
from ..frontend.core import traverse_layer_graph  # noqa: F401
