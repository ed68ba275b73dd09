"""Helpers shared by the graph modules (python/lbann/modules/graph/utils.py): moving between
node-wise and edge-wise tensors."""
from . import GraphExpand, GraphReduce  # noqa: F401
