"""Bookkeeping of the cache on the host: slots, lengths, pages, groups.  No tensors.  The book is a C++ class
(include/qwen3/cache_book.h) behind a C face (csrc/host_runtime.cpp); this module is its binding.

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

import ctypes
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


def _host():
    """The host runtime (include/qwen3/cache_book.h, step_pack.h behind csrc/host_runtime.cpp), loaded once."""
    global _lib
    if _lib is None:
        from ..csrc.build import load_library
        lib = load_library("host_runtime.cpp")
        i32p, i64p = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
        lib.q3_host_last_error.restype = ctypes.c_char_p
        lib.q3_book_create.argtypes = [i32p, i32p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                       ctypes.POINTER(ctypes.c_void_p)]
        lib.q3_book_destroy.argtypes = [ctypes.c_void_p]
        lib.q3_book_destroy.restype = None
        lib.q3_book_info.argtypes = [ctypes.c_void_p, i32p]
        lib.q3_book_info.restype = ctypes.c_int64
        lib.q3_book_alloc_slot.argtypes = [ctypes.c_void_p, i32p]
        lib.q3_book_free_slot.argtypes = [ctypes.c_void_p, ctypes.c_int]
        for name in ("q3_book_reserve", "q3_book_commit", "q3_book_cancel"):
            getattr(lib, name).argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        lib.q3_book_lengths.argtypes = [ctypes.c_void_p]
        lib.q3_book_lengths.restype = i64p
        lib.q3_book_is_held.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.q3_book_free_slots.argtypes = [ctypes.c_void_p]
        lib.q3_book_pages_held.argtypes = [ctypes.c_void_p]
        lib.q3_book_table.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.q3_book_table.restype = i32p
        lib.q3_book_free_pages.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.q3_step_layout.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p]
        lib.q3_pack_step.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64,
                                     ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.q3_pack_decode_step.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                            ctypes.c_void_p]
        _lib = lib
    return _lib


_lib = None


def _raise(code: int) -> None:
    message = _host().q3_host_last_error().decode("utf-8", "replace")
    raise {1: CacheError, 2: CacheFull}.get(code, RuntimeError)(message)


class _Slots:
    """The slots of a book: which are held, how many are free."""

    def __init__(self, book: "CacheBook"):
        self._book = book

    def is_held(self, slot: int) -> bool:
        return bool(_host().q3_book_is_held(self._book._handle, int(slot)))

    @property
    def n_free(self) -> int:
        return int(_host().q3_book_free_slots(self._book._handle))

    @property
    def held(self):
        return frozenset(s for s in range(self._book.n_slots) if self.is_held(s))


class PageGroup:
    """The pages of the layers that share one `CacheNeed`: a view of the book's group."""

    def __init__(self, book: "CacheBook", index: int, need: CacheNeed, layers: List[int]):
        self._book, self._index, self.need, self.layers = book, index, need, layers
        self.n_pages = book.n_pages
        pointer = _host().q3_book_table(book._handle, index)
        self.table = np.ctypeslib.as_array(pointer, shape=(book.n_slots, book.pages_per_slot))   # -1: no page

    @property
    def _free(self) -> List[int]:
        out = np.empty(self.n_pages, dtype=np.int32)
        n = _host().q3_book_free_pages(self._book._handle, self._index, out.ctypes.data)
        return [int(p) for p in out[:n]]

    @property
    def n_free(self) -> int:
        return int(_host().q3_book_free_pages(self._book._handle, self._index, None))

    def held_pages(self, slot: int) -> List[int]:
        row = self.table[slot]
        return [int(p) for p in row[row >= 0]]


class CacheBook:
    """Slots, lengths and pages of every group; the storage class adds the tensors.  The book itself is the
    C++ class of include/qwen3/cache_book.h; this is its binding.

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
        self.group_of_layer: Dict[int, int] = {}
        self.state_layers: Dict[int, Tuple[int, ...]] = {}
        by_key: Dict[tuple, int] = {}
        group_needs: List[CacheNeed] = []
        group_layers: List[List[int]] = []
        for layer, need in enumerate(needs):
            if need is None:
                continue
            if need.state_shape:
                self.state_layers[layer] = tuple(need.state_shape)
            if need.kind == "none":
                continue
            key = need.group_key()
            if key not in by_key:
                by_key[key] = len(group_needs)
                group_needs.append(need)
                group_layers.append([])
            group_layers[by_key[key]].append(layer)
            self.group_of_layer[layer] = by_key[key]
        G = len(group_needs)
        kinds = (ctypes.c_int32 * max(G, 1))(*[1 if n.kind == "window" else 0 for n in group_needs])
        windows = (ctypes.c_int32 * max(G, 1))(*[int(n.window or 0) for n in group_needs])
        handle = ctypes.c_void_p()
        code = _host().q3_book_create(kinds, windows, G, int(max_tokens), int(max_seq_len), int(n_slots or 0), PAGE_TOKENS,
                                      ctypes.byref(handle))
        if code:
            _raise(code)
        self._handle = handle
        info = (ctypes.c_int32 * 5)()
        self.max_seq_len = int(_host().q3_book_info(self._handle, info))
        self.n_pages, self.n_slots, self.pages_per_slot = int(info[0]), int(info[1]), int(info[2])
        self.lengths = np.ctypeslib.as_array(_host().q3_book_lengths(self._handle), shape=(self.n_slots,))
        self.slots = _Slots(self)
        self.groups: List[PageGroup] = [PageGroup(self, g, group_needs[g], group_layers[g]) for g in range(G)]

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle and _lib is not None:
            self.groups, self.lengths = [], None          # the views die with the book
            _lib.q3_book_destroy(handle)

    # -- slots
    def alloc_slot(self) -> int:
        slot = ctypes.c_int32()
        code = _host().q3_book_alloc_slot(self._handle, ctypes.byref(slot))
        if code:
            _raise(code)
        self._on_alloc(slot.value)
        return int(slot.value)

    def free_slot(self, slot: int) -> None:
        code = _host().q3_book_free_slot(self._handle, int(slot))
        if code:
            _raise(code)

    def length(self, slot: int) -> int:
        return int(self.lengths[slot])

    def _on_alloc(self, slot: int) -> None:  # the storage class zeroes the state rows here
        pass

    # -- a step: reserve for every sequence, run, commit (or cancel)
    @staticmethod
    def _arrays(step: Sequence[Tuple[int, int]]):
        slots = np.fromiter((s for s, _ in step), dtype=np.int32, count=len(step))
        n_new = np.fromiter((n for _, n in step), dtype=np.int64, count=len(step))
        return slots, n_new

    def reserve(self, step: Sequence[Tuple[int, int]]) -> None:
        """Make room for `n_new` tokens on each `(slot, n_new)`; nothing changes if it cannot be done."""
        slots, n_new = self._arrays(step)
        code = _host().q3_book_reserve(self._handle, slots.ctypes.data, n_new.ctypes.data, len(step))
        if code:
            _raise(code)

    def cancel(self, step: Sequence[Tuple[int, int]]) -> None:
        """The step did not run after all (its launch failed): the pages that `reserve` took for it go back,
        lengths stay as they were.  What the failed step may have written lies beyond every length."""
        slots, n_new = self._arrays(step)
        code = _host().q3_book_cancel(self._handle, slots.ctypes.data, n_new.ctypes.data, len(step))
        if code:
            _raise(code)

    def commit(self, step: Sequence[Tuple[int, int]]) -> None:
        """The step ran: lengths advance once, window groups return dead pages."""
        slots, n_new = self._arrays(step)
        code = _host().q3_book_commit(self._handle, slots.ctypes.data, n_new.ctypes.data, len(step))
        if code:
            _raise(code)

    # -- views for a step
    def page_rows(self, group: int, slots: Sequence[int]) -> np.ndarray:
        """[len(slots), pages_per_slot] page numbers (-1: none) of one group."""
        return self.groups[group].table[np.asarray(slots, dtype=np.int64)]

    def pages_held(self) -> int:
        """Pages in use in the fullest group: what counts against `max_tokens`."""
        return int(_host().q3_book_pages_held(self._handle))

    # -- the metadata of a step, packed by the host runtime (include/qwen3/step_pack.h)
    def step_layout(self, n_tokens: int, n_seqs: int, n_want: int) -> Tuple[List[int], int]:
        """Offsets of the sections token_ids, token_seq, token_pos, seq_slots, seq_start, seq_pos0, want_rows and of
        one page table per group in a step's int32 buffer, and the buffer's size."""
        G = len(self.groups)
        offsets = (ctypes.c_int32 * (7 + G))()
        total = _host().q3_step_layout(int(n_tokens), int(n_seqs), int(n_want), G, self.pages_per_slot, offsets)
        return [int(o) for o in offsets], int(total)

    def pack_step(self, slots: np.ndarray, n_new: np.ndarray, token_ids: np.ndarray, want_rows: np.ndarray, out: np.ndarray) -> None:
        """Fill `out` (int32, the size `step_layout` gives) for the step; `reserve` has run, `commit` has not."""
        code = _host().q3_pack_step(self._handle, slots.ctypes.data, n_new.ctypes.data, len(slots), token_ids.ctypes.data,
                                    int(token_ids.size), want_rows.ctypes.data, int(want_rows.size), out.ctypes.data)
        if code:
            _raise(code)

    def pack_decode_step(self, rows: int, slots: np.ndarray, token_ids: np.ndarray, out: np.ndarray) -> None:
        """The same for a decode step of a fixed number of `rows`, the rows beyond len(slots) being padding."""
        code = _host().q3_pack_decode_step(self._handle, int(rows), slots.ctypes.data, len(slots), token_ids.ctypes.data,
                                           out.ctypes.data)
        if code:
            _raise(code)
