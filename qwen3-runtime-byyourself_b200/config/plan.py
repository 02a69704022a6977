"""Architecture-independent description of a model: which parts, in which order.

A configuration class (one per architecture) turns its config.json into a
`ModelPlan`.  Everything below the plan - parts, cache, step function, replay,
generation - reads the plan only and never the architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part by the name it was registered under, with its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement that holds a mixer and a feed-forward.

    `prefix` is the checkpoint-name prefix of the layer's tensors.  `cache_from`
    names another layer whose cache this layer's mixer reads instead of owning
    one (None: the layer owns its cache).
    """
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    prefix: str
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    """The whole model as data.

    `order` is the sequence in which layers run; it may name a layer twice.
    """
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    embedding_prefix: str
    layers: List[LayerSpec]
    order: List[int]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
    stop_token_ids: List[int] = field(default_factory=list)

    def __post_init__(self):
        n = len(self.layers)
        for i in self.order:
            if not 0 <= i < n:
                raise ValueError(f"order names layer {i}, but the plan has {n} layers")
        for i, layer in enumerate(self.layers):
            src = layer.cache_from
            if src is None:
                continue
            if not 0 <= src < n or src == i or self.layers[src].cache_from is not None:
                raise ValueError(f"layer {i}: cache_from={src} must name another layer that owns its cache")
            if src not in self.order or i not in self.order or self.order.index(src) > self.order.index(i):
                raise ValueError(f"layer {i} reads the cache of layer {src}, which has to run first")
