"""Models whose branches run on sub-grids of a trainer (python/lbann/models/subgraph)."""
from .transformer import (TransformerAllSubgraph, TransformerDecoderLayerAllSubGraph,  # noqa: F401
                          TransformerEncoderLayerAllSubGraph)
