"""Registries of parts, and what each kind of part has to offer.

A model is put together from parts that are looked up by the `kind` of a `PartSpec`
and built from its `params`.  No part knows which model it is in: sizes, constants
and checkpoint names all arrive as parameters.

Interfaces (duck-typed; `Part` gives the defaults):

  every part      weight_specs(prefix) -> {checkpoint name: WeightSpec}
                  bind(weights, prefix, dtype, device)   takes its tensors from `weights`
  norm            __call__(x, out, delta=None): if delta is given, x += delta in place
                  (32-bit sum) first; out = norm(x).  Rows are the last dimension.
  position        prepare(max_positions, device); apply_(q, k, positions) rotates
                  [N, heads, d] tensors in place.  A rotary encoding also exposes its
                  `cos`/`sin` tables so that the attention kernel can fuse the rotation.
  mixer           cache_need() -> CacheNeed;  forward(x, ctx, cache) -> [N, hidden].
                  `ctx` is the step's StepContext (tokens, positions, sequences, page
                  tables, scratch buffers); `cache` is the layer's LayerCache (pages
                  and/or fixed-size state rows indexed by slot).
  feed_forward    forward(x, ctx) -> [N, hidden]
  block           built from (spec params, mixer, feed_forward); weight_specs/bind cover
                  its own norms; forward(residual, delta, ctx, cache) -> (residual, delta):
                  the hidden state is residual + delta, the sum is left to the next norm.
  embedding       forward(token_ids, out) -> [N, hidden]
  head            forward(x, out) -> float32 logits [R, vocab]
"""
from __future__ import annotations

from typing import Callable, Dict

from ..config.plan import PartSpec

NORMS: Dict[str, Callable] = {}
POSITIONS: Dict[str, Callable] = {}
MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}
EMBEDDINGS: Dict[str, Callable] = {}
HEADS: Dict[str, Callable] = {}

_ALL = {"norm": NORMS, "position": POSITIONS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS, "block": BLOCKS,
        "embedding": EMBEDDINGS, "head": HEADS}


def register_part(family: str, kind: str, factory: Callable) -> None:
    """Make `factory(**params)` the builder of parts of `kind` in `family`
    (norm, position, mixer, feed_forward, block, embedding, head)."""
    _ALL[family][kind] = factory


def build_part(family: str, spec: PartSpec, *args):
    registry = _ALL[family]
    if spec.kind not in registry:
        raise KeyError(f"no {family} part named {spec.kind!r}; registered: {sorted(registry)}")
    return registry[spec.kind](*args, **spec.params)


class Part:
    def weight_specs(self, prefix: str) -> dict:
        return {}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        pass
