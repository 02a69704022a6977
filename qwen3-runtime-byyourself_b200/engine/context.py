"""What a step hands to the parts: the packed tokens, their sequences and positions.

All sequences of a step are packed into one list of N tokens.  The integer metadata
lives in ONE device buffer filled by one host-to-device copy per step; the fields
below are views of it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch


class Scratch:
    """Named activation buffers that are reused from step to step (grown when needed).

    With `guard` (a debugging aid for tests): every buffer has exactly the size asked for and lies between two
    guard zones of 256 bytes filled with a pattern; `violations()` names the buffers whose zones were written."""

    GUARD_BYTES, GUARD_VALUE = 256, 0xA5

    def __init__(self, device, guard: bool = False):
        self.device = torch.device(device)
        self.guard = guard
        self._flat: Dict[Tuple, torch.Tensor] = {}
        self._raw: Dict[Tuple, torch.Tensor] = {}

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        if self.guard:
            return self._guarded(name, numel, dtype).view(*shape)
        key = (name, dtype)
        flat = self._flat.get(key)
        if flat is None or flat.numel() < numel:
            flat = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._flat[key] = flat
        return flat[:numel].view(*shape)

    def _guarded(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, dtype, numel)
        flat = self._flat.get(key)
        if flat is None:
            g = self.GUARD_BYTES
            nbytes = numel * torch.empty((), dtype=dtype).element_size()
            raw = torch.full((g + nbytes + g,), self.GUARD_VALUE, dtype=torch.uint8, device=self.device)
            self._raw[key] = raw
            flat = self._flat[key] = raw[g:g + nbytes].view(dtype)
        return flat

    def violations(self) -> list:
        """Names (with type and size) of guarded buffers whose guard zones no longer hold the pattern."""
        g, bad = self.GUARD_BYTES, []
        for key, raw in self._raw.items():
            if not (bool((raw[:g] == self.GUARD_VALUE).all()) and bool((raw[-g:] == self.GUARD_VALUE).all())):
                bad.append(key)
        return bad


@dataclass
class StepContext:
    n_tokens: int                 # N: tokens in this step, over all sequences
    n_seqs: int                   # B
    n_want: int                   # R: rows whose logits are wanted
    is_decode: bool               # every sequence brings exactly one token
    max_new: int                  # most tokens one sequence brings
    max_context: int              # longest sequence after this step
    max_positions: int            # the engine's bound on a sequence's length
    dtype: torch.dtype
    device: torch.device
    scratch: Scratch
    token_ids: torch.Tensor       # [N] int32
    token_seq: torch.Tensor       # [N] int32: index of the token's sequence within the step
    token_pos: torch.Tensor       # [N] int32: absolute position of the token in its sequence
    seq_slots: torch.Tensor       # [B] int32: cache slot of each sequence
    seq_start: torch.Tensor       # [B + 1] int32: first packed token of each sequence
    seq_pos0: torch.Tensor        # [B] int32: tokens already cached before the step
    want_rows: torch.Tensor       # [R] int32: packed token rows whose logits are wanted
    want_all: bool = False        # every packed row is wanted, in order (R == N): nothing to gather
    page_tables: List[torch.Tensor] = field(default_factory=list)   # per cache group [B, pages_per_slot] int32
    host_slots: List[int] = field(default_factory=list)
    host_n_new: List[int] = field(default_factory=list)
    host_pos0: List[int] = field(default_factory=list)
