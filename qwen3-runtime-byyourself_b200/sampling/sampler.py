"""Chooses the next token of every row on the GPU and brings back only the ids.

Greedy: the argmax kernel.  Sample: the temperature / top-k / top-p kernel, with one
random stream per sequence keyed by (seed, sequence id, step).  The reference's
sampler copies the logits to the host and walks them there
(src/generation/sampler.cpp:277-313); its options and their meaning are kept.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..csrc import ops
from .params import SamplingParams


class NonFiniteLogits(RuntimeError):
    """A row of logits held NaN or Inf (the reference refuses such rows too)."""


class PendingChoice:
    """Ids that are being chosen on the device and copied to the host; `result()` waits for them."""

    def __init__(self, device_ids: torch.Tensor, host_ids: torch.Tensor, event: torch.cuda.Event):
        self.device_ids, self._host, self._event = device_ids, host_ids, event

    def result(self) -> List[int]:
        self._event.synchronize()
        ids = self._host.tolist()
        if any(i < 0 for i in ids):
            raise NonFiniteLogits("sampling met a non-finite logit")
        return ids


class Sampler:
    def __init__(self, params: SamplingParams, vocab_size: int, device):
        if params.valid_vocab_size > vocab_size:
            raise ValueError("valid_vocab_size exceeds logits vocabulary size")
        if params.mode == "sample" and params.top_k > vocab_size:
            raise ValueError("top_k exceeds the vocabulary size")
        self.params, self.vocab_size, self.device = params, vocab_size, torch.device(device)
        self._cap = 0
        self._grow(8)

    def _grow(self, rows: int) -> None:
        if rows <= self._cap:
            return
        self._cap = max(rows, 2 * self._cap)
        self._turn = 0
        self._outs = [torch.empty(self._cap, dtype=torch.int32, device=self.device) for _ in range(2)]
        self._out_hosts = [torch.empty(self._cap, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._out = self._outs[0]
        # stream keys go through pinned staging; one set per turn, since two choices can be in flight
        self._ids_devs = [torch.empty(self._cap, dtype=torch.int64, device=self.device) for _ in range(2)]
        self._steps_devs = [torch.empty(self._cap, dtype=torch.int32, device=self.device) for _ in range(2)]
        self._ids_hosts = [torch.empty(self._cap, dtype=torch.int64).pin_memory() for _ in range(2)]
        self._steps_hosts = [torch.empty(self._cap, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._out_host = torch.empty(self._cap, dtype=torch.int32).pin_memory()
        self._ids_on_device = [None, None]

    def choose_device(self, logits: torch.Tensor, sequence_ids: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """int32 ids [rows] on the device; `sequence_ids[r]`/`steps[r]` key row r's random stream."""
        rows = logits.shape[0]
        self._grow(rows)
        valid = self.params.valid_vocab_size or logits.shape[1]
        out = self._out[:rows]
        if self.params.mode == "greedy":
            return ops.argmax(logits, out, valid)
        t = self._turn
        ids_key = tuple(sequence_ids)
        if self._ids_on_device[t] != ids_key:                # the same sequences as last time: nothing to upload
            self._ids_hosts[t][:rows] = torch.as_tensor(ids_key, dtype=torch.int64)
            self._ids_devs[t][:rows].copy_(self._ids_hosts[t][:rows], non_blocking=True)
            self._ids_on_device[t] = ids_key
        steps = list(steps)
        if all(s == steps[0] for s in steps):                 # sequences that started together: one number
            step_arg = int(steps[0])
        else:
            self._steps_hosts[t][:rows] = torch.as_tensor(steps, dtype=torch.int32)
            self._steps_devs[t][:rows].copy_(self._steps_hosts[t][:rows], non_blocking=True)
            step_arg = self._steps_devs[t][:rows]
        p = self.params
        return ops.sample(logits, out, p.temperature, p.top_k, p.top_p, p.seed, self._ids_devs[t][:rows], step_arg, valid)

    def choose_async(self, logits: torch.Tensor, sequence_ids: Sequence[int], steps: Sequence[int]) -> PendingChoice:
        """Start the choice and its copy to the host without waiting.  Two results can be in flight: the
        device ids of one call stay valid until the call after the next."""
        rows = logits.shape[0]
        self._grow(rows)
        self._turn ^= 1
        self._out = self._outs[self._turn]
        ids = self.choose_device(logits, sequence_ids, steps)
        host = self._out_hosts[self._turn][:rows]
        host.copy_(ids, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingChoice(ids, host, event)

    def choose(self, logits: torch.Tensor, sequence_ids: Sequence[int], steps: Sequence[int]) -> List[int]:
        """The chosen ids as Python ints (one device-to-host copy of 4 bytes per row)."""
        rows = logits.shape[0]
        out = self.choose_device(logits, sequence_ids, steps)
        self._out_host[:rows].copy_(out, non_blocking=False)
        ids = self._out_host[:rows].tolist()
        if any(i < 0 for i in ids):
            raise NonFiniteLogits("sampling met a non-finite logit")
        return ids
