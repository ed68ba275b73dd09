"""Multi-head attention whose heads run on sub-grids of the trainer
(python/lbann/modules/attention_allsubgraph.py): the same module as
``lbann.modules.MultiheadAttention`` with ``subgraph_branches`` set, so that head h lives on
sub-grid 1 + h // (heads / branches) and only the output projection spans all ranks."""
from __future__ import annotations

from .transformer import MultiheadAttention


class MultiheadAttentionAllSubGraph(MultiheadAttention):
    def __init__(self, embed_dim, num_heads, branches, **kwargs):
        if branches < 1 or num_heads % branches:
            raise ValueError(f"{num_heads} heads cannot be dealt to {branches} sub-grids")
        super().__init__(embed_dim, num_heads, subgraph_branches=branches, **kwargs)
