"""The generation loop above the step function.

Requests are taken in order, as many at a time as the cache holds; the prompts of a
batch run in one step, then every live sequence advances by one token a step; a
sequence that draws a stop token or reaches its budget leaves the batch and gives its
slot back; when the batch is empty the next one starts.  No request joins a batch
that has started.

Per sequence the loop is the reference's (src/generation/generator.cpp:249-323):
  logits of the last position -> choose -> record -> stop check -> next step,
  the stop token is recorded and not fed back (:294-301), no step runs after the
  last wanted token (:305-307), max_new_tokens == 0 returns before any step
  (:258-260), an empty prompt is an error (:85-89), prompt + max_new_tokens must fit
  the context (:163-184), stop ids must lie in the vocabulary (:186-195).
The reference generates at batch 1 only (:79-83).

The decisions - which requests may run, the batches, who goes on after a token and why the others
ended - are the host runtime's (include/qwen3/generation.h, C++); this module binds them and drives
the engine and the chooser with them.

The loop needs of its engine only: `new_sequence()`, `release(slot)`,
`step(entries) -> logits`, `max_seq_len`, `vocab_size`, and `cache.n_pages`,
`cache.n_slots`, `cache.page_tokens`; and of its chooser `choose(logits, sequence_ids,
steps) -> ids`.  The tests drive it with stand-ins on the CPU.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import numpy as np

from .engine import StepEntry

MAX_NEW_TOKENS = "max_new_tokens"
STOP_TOKEN = "stop_token"
_REASONS = {1: MAX_NEW_TOKENS, 2: STOP_TOKEN}        # qwen3::StopReason
_lib = None


def _host():
    """The host runtime's generation entry points (csrc/host_runtime.cpp), bound once."""
    global _lib
    if _lib is None:
        from ..cache.book import _host as load
        lib = load()
        p, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        lib.q3_generation_check.argtypes = [p, i, i64, i64, p, i, i64]
        lib.q3_generation_plan_batches.argtypes = [p, i, i64, i64, i, i, i, p]
        lib.q3_progress_create.argtypes = [i, i64, p, i, ctypes.POINTER(p)]
        lib.q3_progress_destroy.argtypes = [p]
        lib.q3_progress_destroy.restype = None
        lib.q3_progress_record.argtypes = [p, p, p, i, p, p]
        lib.q3_progress_may_run_ahead.argtypes = [p, i]
        _lib = lib
    return _lib


def _check(code: int) -> None:
    if code:
        message = _host().q3_host_last_error().decode("utf-8", "replace")
        raise (ValueError if code == 4 else RuntimeError)(message)


class _Progress:
    """qwen3::GenerationProgress: what has been generated for the requests of one call, and who still runs."""

    def __init__(self, n_requests: int, max_new_tokens: int, stops: Sequence[int]):
        stops = np.asarray(sorted(stops), dtype=np.int32)
        handle = ctypes.c_void_p()
        _check(_host().q3_progress_create(n_requests, max_new_tokens, stops.ctypes.data, len(stops), ctypes.byref(handle)))
        self._handle = handle

    def __del__(self):
        if getattr(self, "_handle", None) and _lib is not None:
            _lib.q3_progress_destroy(self._handle)
            self._handle = None

    def record(self, requests: Sequence[int], tokens: Sequence[int]):
        """(goes on?, why it ended) for each request after the token chosen for it."""
        n = len(requests)
        req, tok = np.asarray(requests, dtype=np.int32), np.asarray(tokens, dtype=np.int32)
        on, why = np.empty(n, dtype=np.int32), np.empty(n, dtype=np.int32)
        _check(_host().q3_progress_record(self._handle, req.ctypes.data, tok.ctypes.data, n, on.ctypes.data, why.ctypes.data))
        return [bool(v) for v in on], [_REASONS.get(int(v)) for v in why]

    def may_run_ahead(self, request: int) -> bool:
        return bool(_host().q3_progress_may_run_ahead(self._handle, int(request)))


@dataclass
class GenerationResult:
    """New tokens only (a stop token included), and why the sequence ended."""
    token_ids: List[int] = field(default_factory=list)
    stop_reason: str = MAX_NEW_TOKENS


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, n_pages: int, n_slots: int, page_tokens: int,
                 batch_size: Optional[int] = None) -> List[List[int]]:
    """Split request indices, in order, into batches whose worst-case page need fits the cache."""
    lengths = np.asarray(list(prompt_lengths), dtype=np.int64)
    batch_of = np.empty(len(lengths), dtype=np.int32)
    _check(_host().q3_generation_plan_batches(lengths.ctypes.data, len(lengths), int(max_new_tokens), int(n_pages), int(n_slots),
                                              int(page_tokens), int(batch_size or 0), batch_of.ctypes.data))
    batches: List[List[int]] = []
    for i, b in enumerate(batch_of):
        if b == len(batches):
            batches.append([])
        batches[b].append(i)
    return batches


def generate(engine, prompts: Sequence[Sequence[int]], chooser, max_new_tokens: int = 128,
             stop_token_ids: Sequence[int] = (), batch_size: Optional[int] = None,
             on_token: Optional[Callable[[int, int], None]] = None,
             sequence_ids: Optional[Sequence[int]] = None) -> List[GenerationResult]:
    """Generate for every prompt; `chooser.choose(logits, sequence_ids, steps)` picks the tokens.

    `on_token(request index, token id)` is called for every new token as it is chosen.
    `sequence_ids[i]` names request i to the chooser (its random stream is keyed by it); by default
    a request is named by its index, so the same prompt draws other tokens at another place of the
    list unless it is given the same name."""
    prompts = [list(p) for p in prompts]
    stops = sorted(set(int(t) for t in stop_token_ids))
    lengths, stop_ids = np.asarray([len(p) for p in prompts], dtype=np.int64), np.asarray(stops, dtype=np.int64)
    if stop_ids.size and (stop_ids.min() < -2 ** 31 or stop_ids.max() >= 2 ** 31):
        raise ValueError("a stop token id is outside the vocabulary")
    stop_ids = stop_ids.astype(np.int32)
    _check(_host().q3_generation_check(lengths.ctypes.data, len(prompts), int(max_new_tokens), int(engine.max_seq_len),
                                       stop_ids.ctypes.data, len(stops), int(engine.vocab_size)))
    if sequence_ids is None:
        names = list(range(len(prompts)))
    else:
        names = [int(s) for s in sequence_ids]
        if len(names) != len(prompts):
            raise ValueError("sequence_ids must name every prompt")
    results = [GenerationResult() for _ in prompts]
    if max_new_tokens == 0 or not prompts:
        return results
    cache = engine.cache
    progress = _Progress(len(prompts), max_new_tokens, stops)
    if hasattr(chooser, "choose_async") and getattr(engine, "device_tokens", False):
        for batch in plan_batches([len(p) for p in prompts], max_new_tokens, cache.n_pages, cache.n_slots,
                                  cache.page_tokens, batch_size):
            _run_batch_pipelined(engine, chooser, batch, prompts, results, progress, on_token, names)
        return results
    for batch in plan_batches([len(p) for p in prompts], max_new_tokens, cache.n_pages, cache.n_slots,
                              cache.page_tokens, batch_size):
        live = [(i, engine.new_sequence()) for i in batch]
        try:
            feed = {i: prompts[i] for i, _ in live}
            step_index = 0
            while live:
                entries = [StepEntry(slot, feed[i], [len(feed[i]) - 1]) for i, slot in live]
                logits = engine.step(entries)
                chosen = chooser.choose(logits, [names[i] for i, _ in live], [step_index] * len(live))
                if step_index % 32 == 0 and hasattr(engine, "check_kernels"):
                    engine.check_kernels()            # now and then: a kernel whose bounded wait ran out is reported
                chosen = [int(t) for t in chosen]
                goes_on, why = progress.record([i for i, _ in live], chosen)
                still = []
                for (i, slot), token, on, reason in zip(live, chosen, goes_on, why):
                    results[i].token_ids.append(token)
                    if on_token is not None:
                        on_token(i, token)
                    if on:
                        feed[i] = [token]
                        still.append((i, slot))
                    else:
                        results[i].stop_reason = reason
                        engine.release(slot)
                live = still
                step_index += 1
            if hasattr(engine, "check_kernels"):
                engine.check_kernels()
        except BaseException:
            for _, slot in live:
                try:
                    engine.release(slot)
                except Exception:
                    pass
            raise
    return results


def _run_batch_pipelined(engine, chooser, batch, prompts, results, progress, on_token, names) -> None:
    """One batch with the host one step behind the device.

    The next step is launched before the ids of the current one have reached the host: it reads
    them on the device, where the sampler wrote them, for every sequence that still has budget.  A
    sequence whose pending token turns out to be a stop token has then run one step too many; that
    row is dropped, and its slot goes back like any other.  So the device never waits for the host
    to look at a token, and the decisions are those of the plain loop."""
    from ..cache.book import CacheFull
    live = [(i, engine.new_sequence()) for i in batch]
    ended = set()
    try:
        logits = engine.step([StepEntry(slot, prompts[i], [len(prompts[i]) - 1]) for i, slot in live])
        pending = chooser.choose_async(logits, [names[i] for i, _ in live], [0] * len(live))
        step_index = 0
        while live:
            onward = [(i, slot) for i, slot in live if i not in ended and progress.may_run_ahead(i)]
            upcoming = None
            if onward:
                rows = [k for k, (i, _) in enumerate(live) if (i, _) in onward]
                tokens_on_device = pending.device_ids
                if rows != list(range(len(live))):
                    tokens_on_device = _take(tokens_on_device, rows)
                try:
                    logits = engine.step([StepEntry(slot, [0], [0]) for _, slot in onward],
                                         device_tokens=tokens_on_device)
                    upcoming = chooser.choose_async(logits, [names[i] for i, _ in onward], [step_index + 1] * len(onward))
                except CacheFull:
                    upcoming = None            # no room to run ahead: fall back to waiting for the ids first
            chosen = pending.result()
            if step_index % 32 == 0 and hasattr(engine, "check_kernels"):
                engine.check_kernels()
            fresh = [(i, slot, int(token)) for (i, slot), token in zip(live, chosen) if i not in ended]
            goes_on, why = progress.record([i for i, _, _ in fresh], [t for _, _, t in fresh])
            for (i, slot, token), on, reason in zip(fresh, goes_on, why):
                results[i].token_ids.append(token)
                if on_token is not None:
                    on_token(i, token)
                if not on:
                    results[i].stop_reason = reason
                    ended.add(i)
                    engine.release(slot)
            step_index += 1
            if onward and upcoming is None:
                onward = [(i, slot) for i, slot in onward if i not in ended]
                if onward:
                    logits = engine.step([StepEntry(slot, [results[i].token_ids[-1]], [0]) for i, slot in onward])
                    upcoming = chooser.choose_async(logits, [names[i] for i, _ in onward], [step_index] * len(onward))
            live, pending = (onward, upcoming) if upcoming is not None else ([], None)
        if hasattr(engine, "check_kernels"):
            engine.check_kernels()
    except BaseException:
        for i, slot in live:
            if i not in ended:
                try:
                    engine.release(slot)
                except Exception:
                    pass
        raise


def _take(ids, rows):
    """ids[rows] for a device tensor (or, for the stand-ins of the tests, an array)."""
    if hasattr(ids, "device") and hasattr(ids, "index_select"):
        import torch
        return ids.index_select(0, torch.as_tensor(rows, dtype=torch.long, device=ids.device))
    return ids[rows]
