"""Graph convolutions on edge lists (python/lbann/modules/graph/sparse)."""
from .. import GatedGraphConv, GCNConv, GraphConv, NNConv, SparseGINConv  # noqa: F401
from .. import SparseGINConv as GINConv  # noqa: F401
