"""Graph convolutions on dense adjacency matrices
(python/lbann/modules/graph/dense/*.py).  Node features are ``[nodes, channels]``, the
adjacency matrix ``[nodes, nodes]``; both products run on the batched tensor-core GEMM."""
from __future__ import annotations

from ..frontend import core as L
from .base import ChannelwiseFullyConnectedModule, Module


class DenseGCNConv(Module):
    """X' = A (X W) + b  (Kipf and Welling 2017; A is expected to be normalised)."""

    global_count = 0

    def __init__(self, input_channels, output_channels, bias=True, name=None):
        super().__init__()
        DenseGCNConv.global_count += 1
        self.name = name or f"Dense_GCN_{DenseGCNConv.global_count}"
        self.fc = ChannelwiseFullyConnectedModule(output_channels, bias=bias, name=self.name + "_weights")

    def forward(self, x, adj):
        return L.MatMul(adj, self.fc(x), name=self.name + "_aggregate")


class DenseGraphConv(Module):
    """X' = X W1 + A X W2  (Morris et al. 2019)."""

    global_count = 0

    def __init__(self, input_channels, output_channels, bias=True, name=None):
        super().__init__()
        DenseGraphConv.global_count += 1
        self.name = name or f"Dense_Graph_{DenseGraphConv.global_count}"
        self.self_fc = ChannelwiseFullyConnectedModule(output_channels, bias=bias, name=self.name + "_self")
        self.nbr_fc = ChannelwiseFullyConnectedModule(output_channels, bias=False, name=self.name + "_nbr")

    def forward(self, x, adj):
        return L.Add(self.self_fc(x), L.MatMul(adj, self.nbr_fc(x)), name=self.name + "_sum")


class GINConv(Module):
    """X' = nn((1 + eps) X + A X)  (Xu et al. 2019) on a dense adjacency matrix."""

    global_count = 0

    def __init__(self, nn_module, eps=0.0, name=None):
        super().__init__()
        GINConv.global_count += 1
        self.name = name or f"GIN_{GINConv.global_count}"
        self.nn, self.eps = nn_module, eps

    def forward(self, x, adj):
        agg = L.Add(L.Scale(x, constant=1.0 + self.eps), L.MatMul(adj, x), name=self.name + "_aggregate")
        return self.nn(agg)
