"""Graph convolutions on dense adjacency matrices
(python/lbann/modules/graph/dense/*.py).  Node features are ``[nodes, channels]``, the
adjacency matrix ``[nodes, nodes]``; both products run on the batched tensor-core GEMM."""
from __future__ import annotations

from ...frontend import core as L
from ..base import ChannelwiseFullyConnectedModule, Module


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


DenseGINConv = GINConv      # the dense-adjacency form under an explicit name


class DenseNNConv(Module):
    """Edge-conditioned convolution on a dense, padded edge tensor (Gilmer et al. 2017;
    python/lbann/modules/graph/dense/DenseNNConv.py):

        x'_i = Theta x_i + sum_j A_ij (x_j . h(e_ij))

    ``edge_features`` is ``[nodes * nodes, edge_channels]`` (row i * nodes + j belongs to the
    pair (i, j)), ``h`` a stack of channel-wise modules that ends with ``in * out`` channels,
    ``adj`` the ``[nodes, nodes]`` adjacency matrix (zero where there is no edge)."""

    global_count = 0

    def __init__(self, sequential_nn, num_nodes, input_channels, output_channels, activation=None, name=None):
        super().__init__()
        DenseNNConv.global_count += 1
        self.name = name or f"Dense_NNConv_{DenseNNConv.global_count}"
        self.nn = list(sequential_nn) if isinstance(sequential_nn, (list, tuple)) else [sequential_nn]
        self.n, self.cin, self.cout = num_nodes, input_channels, output_channels
        self.node_fc = ChannelwiseFullyConnectedModule(output_channels, bias=False, activation=activation,
                                                       name=self.name + "_node_weights")

    def forward(self, x, edge_features, adj):
        n, ci, co = self.n, self.cin, self.cout
        e = edge_features
        for layer in self.nn:
            e = layer(e)
        theta = L.Reshape(e, dims=[n * n, ci, co], name=self.name + "_edge_matrices")
        # x_j for every pair (i, j): the node features repeated for every receiving node i
        xj = L.Reshape(L.Tessellate(L.Reshape(x, dims=[1, n, ci]), dims=[n, n, ci]), dims=[n * n, 1, ci])
        msg = L.Reshape(L.MatMul(xj, theta), dims=[n, n, co], name=self.name + "_messages")
        # sum_j A_ij msg_ij as n products [1, n] x [n, out]
        agg = L.Reshape(L.MatMul(L.Reshape(adj, dims=[n, 1, n]), msg), dims=[n, co],
                        name=self.name + "_aggregate")
        return L.Sum(self.node_fc(x), agg, name=self.name + "_sum")


def GraphExpand(features, indices, name=None):
    """out[e] = features[indices[e]]: node features ``[nodes, F]`` to edge rows ``[edges, F]``
    (python/lbann/modules/graph/utils.py)."""
    GraphExpand.count += 1
    return L.Gather(features, indices, axis=0, name=name or f"graph_expand_{GraphExpand.count}")


def GraphReduce(features, indices, dims, name=None):
    """out[indices[e]] += features[e]: edge rows ``[edges, F]`` summed into ``dims`` =
    ``[nodes, F]``."""
    GraphReduce.count += 1
    return L.Scatter(features, indices, dims=list(dims), axis=0, name=name or f"graph_reduce_{GraphReduce.count}")


GraphExpand.count = 0
GraphReduce.count = 0


class _SparseConv(Module):
    """Graphs as edge lists: ``source_indices[e]`` receives the message that
    ``target_indices[e]`` sends (both ``[edges]``; padding edges carry -1 and are dropped by
    the gather / scatter layers)."""

    global_count = 0

    def _name(self, given, stem):
        type(self).global_count += 1
        return given or f"{stem}_{type(self).global_count}"

    def propagate(self, messages, source_indices, target_indices, channels):
        nbr = GraphExpand(messages, target_indices)
        return GraphReduce(nbr, source_indices, [self.num_nodes, channels])


class GCNConv(_SparseConv):
    """x'_i = sum_{j in N(i)} (W x_j) + b  (python/lbann/modules/graph/sparse/GCNConv.py)."""

    global_count = 0

    def __init__(self, input_channels, output_channels, num_nodes, bias=True, activation=L.Relu, name=None,
                 parallel_strategy=None):
        super().__init__()
        self.name = self._name(name, "GCN")
        self.num_nodes, self.cout = num_nodes, output_channels
        bound = (6.0 / (input_channels + output_channels)) ** 0.5
        ws = [L.Weights(initializer=L.UniformInitializer(min=-bound, max=bound), name=self.name + "_weights")]
        if bias:
            ws.append(L.Weights(initializer=L.ConstantInitializer(value=0.0), name=self.name + "_bias_weights"))
        self.nn = ChannelwiseFullyConnectedModule(output_channels, bias=bias, weights=ws, activation=activation,
                                                  name=self.name + "_FC_layer", parallel_strategy=parallel_strategy)

    def forward(self, x, source_indices, target_indices):
        return self.propagate(self.nn(x), source_indices, target_indices, self.cout)


class GraphConv(_SparseConv):
    """x'_i = W1 x_i + sum_{j in N(i)} W2 x_j  (sparse/GraphConv.py)."""

    global_count = 0

    def __init__(self, input_channels, output_channels, num_nodes, bias=True, activation=L.Relu, name=None,
                 parallel_strategy=None):
        super().__init__()
        self.name = self._name(name, "Graph")
        self.num_nodes, self.cout = num_nodes, output_channels
        self.id_nn = ChannelwiseFullyConnectedModule(output_channels, bias=False, activation=activation,
                                                     name=self.name + "_ID_FC_layer",
                                                     parallel_strategy=parallel_strategy)
        self.mat_nn = ChannelwiseFullyConnectedModule(output_channels, bias=bias, activation=activation,
                                                      name=self.name + "_Message_FC_layer",
                                                      parallel_strategy=parallel_strategy)

    def forward(self, x, source_indices, target_indices):
        agg = self.propagate(self.mat_nn(x), source_indices, target_indices, self.cout)
        return L.Sum(self.id_nn(x), agg, name=self.name + "_sum")


class SparseGINConv(_SparseConv):
    """x'_i = nn((1 + eps) x_i + sum_{j in N(i)} x_j) on an edge list (sparse/GINConv.py)."""

    global_count = 0

    def __init__(self, sequential_nn, input_channels, output_channels, num_nodes, eps=1e-6, name=None):
        super().__init__()
        self.name = self._name(name, "GIN")
        self.nn = list(sequential_nn) if isinstance(sequential_nn, (list, tuple)) else [sequential_nn]
        self.num_nodes, self.cin, self.cout, self.eps = num_nodes, input_channels, output_channels, eps

    def forward(self, x, source_indices, target_indices):
        agg = self.propagate(x, source_indices, target_indices, self.cin)
        h = L.Sum(L.Scale(x, constant=1.0 + self.eps), agg, name=self.name + "_aggregate")
        for layer in self.nn:
            h = layer(h)
        return h


class GatedGraphConv(_SparseConv):
    """``num_layers`` rounds of message passing with a shared GRU update (Li et al. 2016;
    sparse/GatedGraphConv.py): m = sum_{j in N(i)} W_l h_j,  h = GRU(m, h).  Inputs narrower
    than ``output_channels`` are zero-padded."""

    global_count = 0

    def __init__(self, input_channels, output_channels, num_nodes, num_layers=1, name=None):
        super().__init__()
        from ..rnn import ChannelwiseGRU
        if input_channels > output_channels:
            raise ValueError(f"node features ({input_channels}) cannot be wider than the output "
                             f"({output_channels})")
        self.name = self._name(name, "GatedGraphConv")
        self.num_nodes, self.cin, self.cout, self.rounds = num_nodes, input_channels, output_channels, num_layers
        self.rnn = ChannelwiseGRU(num_nodes, output_channels, name=self.name + "_gru")
        self.nns = [ChannelwiseFullyConnectedModule(output_channels, bias=False,
                                                    name=f"{self.name}_message_{i}") for i in range(num_layers)]

    def forward(self, x, source_indices, target_indices):
        if self.cin < self.cout:
            zeros = L.Constant(value=0.0, num_neurons=[self.num_nodes, self.cout - self.cin],
                               name=self.name + "_padding")
            x = L.Concatenation(x, zeros, axis=1, name=self.name + "_padded")
        h = x
        for nn in self.nns:
            m = self.propagate(nn(h), source_indices, target_indices, self.cout)
            h = self.rnn(m, h)
        return h


class NNConv(_SparseConv):
    """Edge-conditioned convolution on an edge list (Gilmer et al. 2017; sparse/NNConv.py):

        x'_i = Theta x_i + sum_{e = (i, j)} x_j . h(edge_features[e])

    ``neighbor_features`` holds x_j per edge as ``[edges, 1, in]`` (``GraphExpand`` of the node
    features by the target indices, reshaped), ``h`` maps ``[edges, 1, edge_in]`` to
    ``[edges, 1, in * out]``; ``edge_index`` names the receiving node of every edge."""

    global_count = 0

    def __init__(self, sequential_nn, num_nodes, num_edges, input_channels, output_channels,
                 edge_input_channels, activation=L.Relu, name=None, parallel_strategy=None):
        super().__init__()
        self.name = self._name(name, "NNConv")
        self.nn = list(sequential_nn) if isinstance(sequential_nn, (list, tuple)) else [sequential_nn]
        self.num_nodes, self.num_edges = num_nodes, num_edges
        self.cin, self.cout, self.ein = input_channels, output_channels, edge_input_channels
        self.node_nn = ChannelwiseFullyConnectedModule(output_channels, bias=False, activation=activation,
                                                       name=self.name + "_node_weights",
                                                       parallel_strategy=parallel_strategy)

    def message(self, node_features, neighbor_features, edge_features):
        x = L.Reshape(node_features, dims=[self.num_nodes, 1, self.cin])
        e = L.Reshape(edge_features, dims=[self.num_edges, 1, self.ein])
        for layer in self.nn:
            e = layer(e)
        theta = L.Reshape(e, dims=[self.num_edges, self.cin, self.cout], name=self.name + "_edge_mat_reshape")
        return self.node_nn(x), L.MatMul(neighbor_features, theta)

    def aggregate(self, edge_values, edge_indices):
        vals = L.Reshape(edge_values, dims=[self.num_edges, self.cout], name=self.name + "_neighbor_features")
        return L.Scatter(vals, edge_indices, dims=[self.num_nodes, self.cout], axis=0,
                         name=self.name + "_aggregate")

    def forward(self, node_features, neighbor_features, edge_features, edge_index):
        own, msgs = self.message(node_features, neighbor_features, edge_features)
        agg = self.aggregate(msgs, edge_index)
        own = L.Reshape(own, dims=[self.num_nodes, self.cout])
        return L.Sum(own, agg, name=self.name + "_sum")
