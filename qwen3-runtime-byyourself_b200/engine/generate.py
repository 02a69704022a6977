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

The loop needs of its engine only: `new_sequence()`, `release(slot)`,
`step(entries) -> logits`, `max_seq_len`, `vocab_size`, and `cache.n_pages`,
`cache.n_slots`, `cache.page_tokens`; and of its chooser `choose(logits, sequence_ids,
steps) -> ids`.  The tests drive it with stand-ins on the CPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from .engine import StepEntry

MAX_NEW_TOKENS = "max_new_tokens"
STOP_TOKEN = "stop_token"


@dataclass
class GenerationResult:
    """New tokens only (a stop token included), and why the sequence ended."""
    token_ids: List[int] = field(default_factory=list)
    stop_reason: str = MAX_NEW_TOKENS


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, n_pages: int, n_slots: int, page_tokens: int,
                 batch_size: Optional[int] = None) -> List[List[int]]:
    """Split request indices, in order, into batches whose worst-case page need fits the cache."""
    batches, current, used = [], [], 0
    for i, n in enumerate(prompt_lengths):
        need = -(-(n + max_new_tokens) // page_tokens)
        if need > n_pages:
            raise ValueError(f"request {i}: {n} prompt + {max_new_tokens} new tokens need {need} pages, "
                             f"the cache has {n_pages}")
        full = len(current) >= n_slots or (batch_size is not None and len(current) >= batch_size)
        if current and (full or used + need > n_pages):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
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
    if max_new_tokens < 0:
        raise ValueError("max_new_tokens cannot be negative")
    stops = set(int(s) for s in stop_token_ids)
    for s in stops:
        if not 0 <= s < engine.vocab_size:
            raise ValueError(f"stop token id {s} is outside the vocabulary")
    prompts = [list(p) for p in prompts]
    for i, p in enumerate(prompts):
        if not p:
            raise ValueError(f"request {i}: the prompt is empty")
        if len(p) + max_new_tokens > engine.max_seq_len:
            raise ValueError(f"request {i}: {len(p)} prompt tokens + {max_new_tokens} new tokens exceed the "
                             f"context of {engine.max_seq_len}")
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
    if hasattr(chooser, "choose_async") and getattr(engine, "device_tokens", False):
        for batch in plan_batches([len(p) for p in prompts], max_new_tokens, cache.n_pages, cache.n_slots,
                                  cache.page_tokens, batch_size):
            _run_batch_pipelined(engine, chooser, batch, prompts, results, max_new_tokens, stops, on_token, names)
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
                still = []
                for (i, slot), token in zip(live, chosen):
                    token = int(token)
                    results[i].token_ids.append(token)
                    if on_token is not None:
                        on_token(i, token)
                    if token in stops:
                        results[i].stop_reason = STOP_TOKEN
                    elif len(results[i].token_ids) >= max_new_tokens:
                        results[i].stop_reason = MAX_NEW_TOKENS
                    else:
                        feed[i] = [token]
                        still.append((i, slot))
                        continue
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


def _run_batch_pipelined(engine, chooser, batch, prompts, results, max_new_tokens, stops, on_token, names) -> None:
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
            onward = [(i, slot) for i, slot in live if i not in ended and len(results[i].token_ids) + 1 < max_new_tokens]
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
            for (i, slot), token in zip(live, chosen):
                if i in ended:
                    continue
                token = int(token)
                results[i].token_ids.append(token)
                if on_token is not None:
                    on_token(i, token)
                if token in stops:
                    results[i].stop_reason = STOP_TOKEN
                elif len(results[i].token_ids) >= max_new_tokens:
                    results[i].stop_reason = MAX_NEW_TOKENS
                else:
                    continue
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
