"""Graph convolutions on dense adjacency matrices (python/lbann/modules/graph/dense)."""
from .. import DenseGCNConv, DenseGINConv, DenseGraphConv, DenseNNConv  # noqa: F401
