"""Parallelisation switches for the transformer / GPT models.

The same command-line surface as the reference's transformer application
(applications/nlp/transformer/parallelism.py:17-400): sharded-weight data parallelism on the
MLP or on every weight, model (tensor) parallelism on the feed-forward blocks and on the
language-model head, and layer parallelism by grid tags.  The functions act on a finished
``lbann.Model`` and recognise the blocks by the layer and weight names that
``lbann_b200.models.transformer`` emits (``<block>_fc1``, ``<block>_fc2``, ``*_matrix``),
so they work on graphs that were built by any code path and then handed over.
"""
from __future__ import annotations

import argparse
import math
import re
from typing import Iterable, List, Optional

from ..frontend import core as L

_BLOCK = re.compile(r"_(?:block|encoder|decoder)(\d+)_")


def add_transformer_parallelism_arguments(parser: argparse.ArgumentParser, subgraph: bool = True) -> None:
    g = parser.add_argument_group("transformer parallelism")
    g.add_argument("--ffn-parallel", action="store_true",
                   help="model parallelism on the feed-forward blocks")
    g.add_argument("--lm-head-parallel", action="store_true",
                   help="model parallelism from the language-model head to the loss")
    g.add_argument("--fsdp", action="store_true", help="shard the first weight of every layer")
    g.add_argument("--fsdp-mlp", action="store_true", help="shard only the feed-forward weights")
    g.add_argument("--fsdp-ranks", type=int, default=0,
                   help="ranks that share one copy of the sharded weights (0: all ranks); "
                        "also the trainer grid height")
    g.add_argument("--layer-parallel", action="store_true",
                   help="contiguous groups of blocks on separate sub-grids")
    g.add_argument("--lp-count", type=int, default=0, help="number of sub-grids (0: one per rank)")
    if subgraph:
        g.add_argument("--attn-head-parallel", type=int, default=0,
                       help="attention heads split over this many sub-graph branches")


def _strategy(args):
    return L.ShardingStrategy.GRID_ROWS if getattr(args, "fsdp_ranks", 0) > 0 else L.ShardingStrategy.FULL


def _all_weights(model) -> List:
    seen, out = set(), []
    for layer in model.layers:
        for w in layer.weights or []:
            if id(w) not in seen:
                seen.add(id(w))
                out.append(w)
    return out


def apply_fsdp_mlp(model, args, other_weights: Iterable = ()) -> int:
    """Flags the feed-forward matrices (and ``other_weights``, e.g. the embeddings) as
    sharded.  Returns how many weights were flagged."""
    if not getattr(args, "fsdp_mlp", False):
        return 0
    if getattr(args, "ffn_parallel", False):
        raise ValueError("sharded weights cannot be combined with model parallelism")
    n = 0
    for w in list(_all_weights(model)) + list(other_weights):
        if w in other_weights or re.search(r"_fc[12]_matrix$", w.name or ""):
            w.sharded, w.sharding_strategy = True, _strategy(args)
            n += 1
    return n


def apply_fsdp_allweights(model, args) -> int:
    """Flags the first weight of every layer except the layer normalisations (their scale
    and bias are short vectors that are cheaper to replicate)."""
    if not getattr(args, "fsdp", False):
        return 0
    if getattr(args, "ffn_parallel", False):
        raise ValueError("sharded weights cannot be combined with model parallelism")
    n = 0
    for layer in model.layers:
        if type(layer).__name__ == "LayerNorm" or not layer.weights:
            continue
        w = layer.weights[0]
        if not w.sharded:
            w.sharded, w.sharding_strategy = True, _strategy(args)
            n += 1
    return n


def apply_ffn_model_parallelism(model, args, blocks: Optional[List[int]] = None) -> List[str]:
    """Puts the feed-forward layers of the chosen blocks (default: all) into the
    model-parallel layout.  Returns the names of the layers that were changed."""
    if not getattr(args, "ffn_parallel", False):
        return []
    changed = []
    for layer in model.layers:
        name = layer.name or ""
        if not re.search(r"_fc[12](?:_instance\d+)?$", name):
            continue
        m = _BLOCK.search(name)
        if blocks is not None and (m is None or int(m.group(1)) not in blocks):
            continue
        layer.data_layout = "model_parallel"
        changed.append(name)
    return changed


def apply_lm_head_model_parallelism(model, lm_head, args) -> List[str]:
    """Every layer from ``lm_head`` to the end of the graph gets the model-parallel layout."""
    if not getattr(args, "lm_head_parallel", False):
        return []
    reach, frontier = {id(lm_head)}, [lm_head]
    while frontier:
        for c in frontier.pop().children:
            if id(c) not in reach:
                reach.add(id(c))
                frontier.append(c)
    changed = []
    for layer in model.layers:
        if id(layer) in reach:
            layer.data_layout = "model_parallel"
            changed.append(layer.name)
    return changed


def apply_layer_parallelism(model, args, world_size: int = 1) -> int:
    """Contiguous groups of transformer blocks get increasing grid tags (placement only: the
    grids run one after the other within a step, as in the reference), and an Identity on
    the destination grid is inserted on every edge that crosses grids from a layer with
    several children.  Returns the number of grids, to be passed as ``--num-subgrids``."""
    if not getattr(args, "layer_parallel", False):
        return 0
    count = getattr(args, "lp_count", 0) or world_size
    ids = sorted({int(m.group(1)) for l in model.layers for m in [_BLOCK.search(l.name or "")] if m})
    if not ids:
        return 0
    per = math.ceil(len(ids) / max(count, 1))
    tag_of = {b: i // per + 1 for i, b in enumerate(ids)}
    for layer in model.layers:
        m = _BLOCK.search(layer.name or "")
        if m:
            layer.grid_tag = {"value": tag_of[int(m.group(1))]}

    def tag(l):
        return (l.grid_tag or {}).get("value", 0)

    inserts = []
    for i, layer in enumerate(model.layers):
        if len(layer.children) <= 1:
            continue
        by_grid = {}
        for child in layer.children:
            if tag(child) != tag(layer):
                by_grid.setdefault(tag(child), []).append(child)
        for g, kids in by_grid.items():
            relay = L.Identity(layer, grid_tag=g, name=f"{layer.name}_to_grid{g}")
            for child in kids:
                child.parents[child.parents.index(layer)] = relay
                layer.children.remove(child)
                relay.children.append(child)
            inserts.append((i + 1, relay))
    for i, relay in reversed(inserts):
        model.layers.insert(i, relay)
    return max(tag_of.values())


def apply_all(model, args, world_size: int = 1) -> List[str]:
    """Applies every switch that ``args`` carries and returns the extra driver arguments the
    choice needs (``--num_subgrids`` for layer parallelism, ``--trainer_grid_height`` when the
    sharded weights are shared by ``--fsdp-ranks`` ranks or layers are model-parallel)."""
    extra: List[str] = []
    apply_fsdp_mlp(model, args)
    apply_fsdp_allweights(model, args)
    changed = apply_ffn_model_parallelism(model, args)
    grids = apply_layer_parallelism(model, args, world_size)
    if grids:
        extra.append(f"--num_subgrids={grids}")
    height = getattr(args, "fsdp_ranks", 0) or (world_size if changed else 0)
    if height and height > 1:
        extra.append(f"--trainer_grid_height={height}")
    return extra
