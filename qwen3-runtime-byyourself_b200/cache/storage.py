"""The cache's device storage: pages of keys and values per group, state per layer.

Layout of one group: [layer in group, K|V, page, kv head, token in page, head_dim].
A (page, kv head) tile is one contiguous [PAGE_TOKENS, head_dim] panel, so a kernel
streams whole panels and a 2-D bulk copy can fetch one.  State rows are float32
[slot, *state_shape] per layer and are zeroed when the slot is handed out; row number
`n_slots` belongs to no sequence and takes the padding rows of a fixed-size decode batch.  Every group
has one page more than its pool hands out: page number `n_pages` belongs to no
sequence and takes the writes of the padding rows of a fixed-size decode batch.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, Optional, Sequence

import torch

from .book import PAGE_TOKENS, CacheBook, CacheNeed


@dataclass
class LayerCache:
    """What one layer's mixer gets: its pages (None: no keys) and its state rows (None: no state)."""
    group: Optional[int]
    keys: Optional[torch.Tensor]      # [n_pages, num_kv_heads, PAGE_TOKENS, head_dim]
    values: Optional[torch.Tensor]
    state: Optional[torch.Tensor]     # [n_slots, *state_shape] float32
    window: Optional[int] = None
    shared: bool = False              # the view of a layer that reads another layer's cache: it must not write


class KVCache(CacheBook):
    def __init__(self, needs: Sequence[Optional[CacheNeed]], max_tokens: int, max_seq_len: int,
                 dtype: torch.dtype, device, n_slots: Optional[int] = None, cache_from: Optional[Dict[int, int]] = None):
        super().__init__(needs, max_tokens, max_seq_len, n_slots)
        self.dtype, self.device = dtype, torch.device(device)
        self.stores = [
            torch.zeros((len(g.layers), 2, g.n_pages + 1, g.need.num_kv_heads, PAGE_TOKENS, g.need.head_dim),
                        dtype=dtype, device=self.device)
            for g in self.groups]
        self.states = {layer: torch.zeros((self.n_slots + 1,) + shape, dtype=torch.float32, device=self.device)
                       for layer, shape in self.state_layers.items()}
        self._views: Dict[int, LayerCache] = {}
        for layer, need in enumerate(needs):
            if need is None:
                continue
            gi = self.group_of_layer.get(layer)
            keys = values = None
            if gi is not None:
                li = self.groups[gi].layers.index(layer)
                keys, values = self.stores[gi][li, 0], self.stores[gi][li, 1]
            self._views[layer] = LayerCache(gi, keys, values, self.states.get(layer),
                                            need.window if need.kind == "window" else None)
        for layer, src in (cache_from or {}).items():
            self._views[layer] = dataclasses.replace(self._views[src], shared=True)

    def _on_alloc(self, slot: int) -> None:
        for state in self.states.values():
            state[slot].zero_()

    def layer(self, index: int) -> LayerCache:
        return self._views[index]

    def bytes_per_token(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.layers) * 2 * g.need.num_kv_heads * g.need.head_dim * item for g in self.groups)
