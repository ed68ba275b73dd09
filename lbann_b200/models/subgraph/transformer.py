"""Transformer with the attention heads of every layer spread over sub-grids.

The reference keeps a second copy of its Transformer for this
(python/lbann/models/subgraph/transformer.py: ``TransformerEncoderLayerAllSubGraph``,
``TransformerDecoderLayerAllSubGraph``, ``TransformerAllSubgraph``); here the ordinary layers
take the number of branches as a parameter and these names fix it.  ``branches`` heads groups
run on the sub-grids 1..branches (``--num-subgrids branches``); everything else runs on the
whole trainer, and tensors change grids at the head slices and at the concatenation.
"""
from __future__ import annotations

from ..transformer import Transformer, TransformerDecoderLayer, TransformerEncoderLayer


class TransformerEncoderLayerAllSubGraph(TransformerEncoderLayer):
    def __init__(self, branches, embed_dim=512, num_heads=8, **kw):
        super().__init__(embed_dim=embed_dim, num_heads=num_heads, branches=branches, **kw)


class TransformerDecoderLayerAllSubGraph(TransformerDecoderLayer):
    def __init__(self, branches, embed_dim=512, num_heads=8, **kw):
        super().__init__(embed_dim=embed_dim, num_heads=num_heads, branches=branches, **kw)


class TransformerAllSubgraph(Transformer):
    def __init__(self, branches, hidden_size=512, num_heads=8, **kw):
        super().__init__(hidden_size=hidden_size, num_heads=num_heads, branches=branches, **kw)
