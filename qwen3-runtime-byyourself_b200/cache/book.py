"""Bookkeeping of the cache on the host: slots, lengths, pages, groups.  No tensors.

A *slot* belongs to one sequence from its first step until the batch gives it
back.  Keys and values live in *pages* of `PAGE_TOKENS` tokens; a slot holds, for
every layer group, a list of pages that covers its length.  Layers whose mixers
state the same need (`CacheNeed`) form a *group* with a page pool of its own; a
group that needs only a window of keys returns the pages that fell out of the
window after each step.  Per-sequence state of fixed size is kept per layer and
is zeroed when a slot is handed out.

The reference keeps two dense [L, Bmax, Smax, nkv, d] tensors with one length per
layer shared by all batch rows (src/model/kv_cache.cpp:55-74, include/qwen3/model/
kv_cache.h:93-99); its append-only rule (:115-117) and capacity check (:119-123)
are kept here per slot, and `reset` is logical only as there (:206-214).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

PAGE_TOKENS = 64


@dataclass(frozen=True)
class CacheNeed:
    """What one layer's mixer asks of the cache.

    kind 'full': keys and values of every past token; 'window': of the last
    `window` tokens; 'none': no keys.  `state_shape` is a fixed-size float32 area
    per sequence (empty: none); it can go with any kind.
    """
    kind: str = "none"
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()

    def __post_init__(self):
        if self.kind not in ("full", "window", "none"):
            raise ValueError(f"unknown cache kind {self.kind!r}")
        if self.kind == "window" and not (self.window and self.window > 0):
            raise ValueError("a window group needs a positive window")
        if self.kind != "none" and (self.num_kv_heads <= 0 or self.head_dim <= 0):
            raise ValueError("a key/value group needs num_kv_heads and head_dim")

    def group_key(self):
        return (self.kind, self.num_kv_heads, self.head_dim, self.window if self.kind == "window" else None)


class CacheError(RuntimeError):
    """Misuse of the cache: a slot freed twice, a step on a slot that is not held."""


class CacheFull(CacheError):
    """No slot or not enough pages are free for what was asked."""


class SlotAllocator:
    """Hands out slot numbers; a slot is held once and freed once."""

    def __init__(self, n_slots: int):
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._held = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} slots are held")
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def free(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheError(f"slot {slot} is not held (freed twice, or never handed out)")
        self._held.remove(slot)
        self._free.append(slot)

    def is_held(self, slot: int) -> bool:
        return slot in self._held

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def held(self):
        return frozenset(self._held)


class PageGroup:
    """The pages of the layers that share one `CacheNeed`."""

    def __init__(self, need: CacheNeed, layers: List[int], n_pages: int, n_slots: int, pages_per_slot: int):
        self.need, self.layers, self.n_pages = need, layers, n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self.table = np.full((n_slots, pages_per_slot), -1, dtype=np.int32)
        self.first_live = np.zeros(n_slots, dtype=np.int64)   # first page index still held (window groups)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def pages_needed(self, length_now: int, n_new: int) -> int:
        have = -(-length_now // PAGE_TOKENS)
        want = -(-(length_now + n_new) // PAGE_TOKENS)
        return want - have

    def extend(self, slot: int, length_now: int, n_new: int) -> None:
        have = -(-length_now // PAGE_TOKENS)
        want = -(-(length_now + n_new) // PAGE_TOKENS)
        for i in range(have, want):
            self.table[slot, i] = self._free.pop()

    def shrink(self, slot: int, length_now: int, n_new: int) -> None:
        """Undo `extend(slot, length_now, n_new)`: the pages it took go back to the pool."""
        have = -(-length_now // PAGE_TOKENS)
        want = -(-(length_now + n_new) // PAGE_TOKENS)
        for i in range(want - 1, have - 1, -1):
            page = int(self.table[slot, i])
            if page >= 0:
                self._free.append(page)
                self.table[slot, i] = -1

    def trim_window(self, slot: int, length: int) -> None:
        """Give back the pages that no later query of this sequence can read."""
        if self.need.kind != "window":
            return
        # a query at position >= length reads keys > length - window
        dead_pages = max(0, (length - self.need.window + 1) // PAGE_TOKENS)
        for i in range(int(self.first_live[slot]), dead_pages):
            page = int(self.table[slot, i])
            if page >= 0:
                self._free.append(page)
                self.table[slot, i] = -1
        self.first_live[slot] = max(int(self.first_live[slot]), dead_pages)

    def release(self, slot: int) -> None:
        row = self.table[slot]
        for page in row[row >= 0]:
            self._free.append(int(page))
        row[:] = -1
        self.first_live[slot] = 0

    def held_pages(self, slot: int) -> List[int]:
        row = self.table[slot]
        return [int(p) for p in row[row >= 0]]


class CacheBook:
    """Slots, lengths and pages of every group; the storage class adds the tensors.

    `needs[i]` is the need of layer i, or None for a layer that reads another
    layer's cache.  `max_tokens` is the most tokens that live sequences hold at
    any time, each sequence rounded up to whole pages; `max_seq_len` bounds one
    sequence.
    """

    def __init__(self, needs: Sequence[Optional[CacheNeed]], max_tokens: int, max_seq_len: int,
                 n_slots: Optional[int] = None):
        if max_tokens <= 0 or max_seq_len <= 0:
            raise ValueError("max_tokens and max_seq_len must be positive")
        self.page_tokens = PAGE_TOKENS
        self.n_pages = -(-max_tokens // PAGE_TOKENS)
        self.max_seq_len = min(max_seq_len, self.n_pages * PAGE_TOKENS)
        self.pages_per_slot = -(-self.max_seq_len // PAGE_TOKENS)
        self.n_slots = n_slots if n_slots is not None else self.n_pages
        self.slots = SlotAllocator(self.n_slots)
        self.lengths = np.zeros(self.n_slots, dtype=np.int64)
        self.groups: List[PageGroup] = []
        self.group_of_layer: Dict[int, int] = {}
        self.state_layers: Dict[int, Tuple[int, ...]] = {}
        by_key: Dict[tuple, int] = {}
        for layer, need in enumerate(needs):
            if need is None:
                continue
            if need.state_shape:
                self.state_layers[layer] = tuple(need.state_shape)
            if need.kind == "none":
                continue
            key = need.group_key()
            if key not in by_key:
                by_key[key] = len(self.groups)
                self.groups.append(PageGroup(need, [], self.n_pages, self.n_slots, self.pages_per_slot))
            self.groups[by_key[key]].layers.append(layer)
            self.group_of_layer[layer] = by_key[key]

    # -- slots
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        self._on_alloc(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        return int(self.lengths[slot])

    def _on_alloc(self, slot: int) -> None:  # the storage class zeroes the state rows here
        pass

    # -- a step: reserve for every sequence, run, commit
    def reserve(self, step: Sequence[Tuple[int, int]]) -> None:
        """Make room for `n_new` tokens on each `(slot, n_new)`; nothing changes if it cannot be done."""
        seen = set()
        for slot, n_new in step:
            if not self.slots.is_held(slot):
                raise CacheError(f"slot {slot} is not held")
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n_new <= 0:
                raise CacheError(f"slot {slot}: a step needs at least one token")
            if self.lengths[slot] + n_new > self.max_seq_len:
                raise CacheFull(f"slot {slot}: {int(self.lengths[slot])} + {n_new} tokens exceed the "
                                f"sequence capacity {self.max_seq_len}")
        for g in self.groups:
            need = sum(g.pages_needed(int(self.lengths[s]), n) for s, n in step)
            if need > g.n_free:
                raise CacheFull(f"the step needs {need} pages of {PAGE_TOKENS} tokens, {g.n_free} are free "
                                f"(of {g.n_pages})")
        for g in self.groups:
            for slot, n_new in step:
                g.extend(slot, int(self.lengths[slot]), n_new)

    def cancel(self, step: Sequence[Tuple[int, int]]) -> None:
        """The step did not run after all (its launch failed): the pages that `reserve` took for it go back,
        lengths stay as they were.  What the failed step may have written lies beyond every length."""
        for g in self.groups:
            for slot, n_new in step:
                g.shrink(slot, int(self.lengths[slot]), n_new)

    def commit(self, step: Sequence[Tuple[int, int]]) -> None:
        """The step ran: lengths advance once, window groups return dead pages."""
        for slot, n_new in step:
            self.lengths[slot] += n_new
            for g in self.groups:
                g.trim_window(slot, int(self.lengths[slot]))

    # -- views for a step
    def page_rows(self, group: int, slots: Sequence[int]) -> np.ndarray:
        """[len(slots), pages_per_slot] page numbers (-1: none) of one group."""
        return self.groups[group].table[np.asarray(slots, dtype=np.int64)]

    def pages_held(self) -> int:
        """Pages in use in the fullest group: what counts against `max_tokens`."""
        return max((g.n_pages - g.n_free for g in self.groups), default=0)
