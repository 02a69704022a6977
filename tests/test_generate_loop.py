"""The generation loop's decisions, driven on the CPU with a stand-in engine whose logits are
scripted: batching by capacity, unequal prompts, stop tokens, sequences that end earlier,
budgets, the order of tokens fed, slots given back, and the reference's edge cases."""
import numpy as np
import pytest

import qwen3_b200 as q
from qwen3_b200.cache import CacheBook, CacheNeed


class ScriptedEngine:
    """Next token = (sum of the sequence's tokens so far) % vocab, so every decision is checkable."""

    def __init__(self, vocab=50, max_tokens=64 * 6, max_seq_len=128, n_slots=None):
        self.vocab_size, self.max_seq_len = vocab, max_seq_len
        self.cache = CacheBook([CacheNeed("full", 1, 16)], max_tokens, max_seq_len, n_slots)
        self.max_seq_len = self.cache.max_seq_len
        self.sums, self.steps, self.peak_slots = {}, [], 0

    def new_sequence(self):
        slot = self.cache.alloc_slot()
        self.sums[slot] = 0
        self.peak_slots = max(self.peak_slots, len(self.cache.slots.held))
        return slot

    def release(self, slot):
        self.cache.free_slot(slot)
        del self.sums[slot]

    def step(self, entries):
        step = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.reserve(step)
        self.steps.append([(e.slot, list(e.tokens), list(e.want)) for e in entries])
        logits = np.full((len(entries), self.vocab_size), -1.0)
        for r, e in enumerate(entries):
            assert list(e.want) == [len(e.tokens) - 1]
            self.sums[e.slot] += sum(e.tokens)
            logits[r, self.sums[e.slot] % self.vocab_size] = 1.0
        self.cache.commit(step)
        return logits


class Argmax:
    def __init__(self):
        self.calls = []

    def choose(self, logits, sequence_ids, steps):
        self.calls.append((list(sequence_ids), list(steps)))
        return [int(np.argmax(row)) for row in logits]


def expected(prompt, max_new, stops, vocab=50):
    total, out = sum(prompt), []
    for _ in range(max_new):
        t = total % vocab
        out.append(t)
        if t in stops:
            return out, q.STOP_TOKEN
        total += t
    return out, q.MAX_NEW_TOKENS


def test_unequal_prompts_stop_tokens_and_early_ends():
    engine, chooser = ScriptedEngine(), Argmax()
    prompts = [[1, 2, 3], [7], [4, 4, 4, 4, 4, 4, 4], [9, 9]]
    stops = [28, 22]
    results = q.generate(engine, prompts, chooser, max_new_tokens=9, stop_token_ids=stops)
    for p, r in zip(prompts, results):
        want, reason = expected(p, 9, stops)
        assert r.token_ids == want and r.stop_reason == reason
    assert {r.stop_reason for r in results} == {q.STOP_TOKEN, q.MAX_NEW_TOKENS}
    # the prompts ran in one step; afterwards one token each for the sequences still alive
    assert [len(t) for _, t, _ in engine.steps[0]] == [3, 1, 7, 2]
    for step in engine.steps[1:]:
        assert all(len(t) == 1 for _, t, _ in step)
    sizes = [len(s) for s in engine.steps]
    assert sizes == sorted(sizes, reverse=True) and sizes[-1] < sizes[0]
    # no step after the last wanted token; the stop token is not fed back
    assert len(engine.steps) == max(len(r.token_ids) for r in results)
    assert engine.cache.slots.n_free == engine.cache.n_slots and engine.cache.pages_held() == 0
    assert chooser.calls[0] == ([0, 1, 2, 3], [0, 0, 0, 0]) and chooser.calls[1][1][0] == 1


def test_batches_follow_one_another_and_reuse_slots():
    engine = ScriptedEngine(max_tokens=64 * 3, max_seq_len=128)        # three pages
    prompts = [[i + 1] * n for i, n in enumerate([5, 60, 3, 70, 2, 2, 2, 2])]
    results = q.generate(engine, prompts, Argmax(), max_new_tokens=10)
    for p, r in zip(prompts, results):
        assert (r.token_ids, r.stop_reason) == expected(p, 10, [])
    # worst case pages: 1, 2 | 1, 2 | 1, 1, 1 | 1  -> batches of 2, 2, 3, 1
    assert q.plan_batches([len(p) for p in prompts], 10, 3, 3, 64) == [[0, 1], [2, 3], [4, 5, 6], [7]]
    assert engine.peak_slots == 3 and engine.cache.slots.n_free == 3
    first_steps = [s for s in engine.steps if any(len(t) > 1 for _, t, _ in s)]
    assert [len(s) for s in first_steps] == [2, 2, 3, 1]


def test_batch_size_and_slot_limits():
    assert q.plan_batches([1] * 5, 1, 100, 100, 64, batch_size=2) == [[0, 1], [2, 3], [4]]
    assert q.plan_batches([1] * 5, 1, 100, 3, 64) == [[0, 1, 2], [3, 4]]
    with pytest.raises(ValueError, match="pages"):
        q.plan_batches([100], 100, 3, 3, 64)


def test_reference_edge_cases():
    engine = ScriptedEngine()
    assert [r.token_ids for r in q.generate(engine, [[1], [2, 3]], Argmax(), max_new_tokens=0)] == [[], []]
    assert engine.steps == []                                   # nothing ran
    with pytest.raises(ValueError, match="empty"):
        q.generate(engine, [[1], []], Argmax(), max_new_tokens=4)
    with pytest.raises(ValueError, match="context"):
        q.generate(engine, [[1] * 120], Argmax(), max_new_tokens=9)
    with pytest.raises(ValueError, match="vocabulary"):
        q.generate(engine, [[1]], Argmax(), max_new_tokens=4, stop_token_ids=[50])
    with pytest.raises(ValueError):
        q.generate(engine, [[1]], Argmax(), max_new_tokens=-1)
    # a stop token as the very first choice: one token, one step
    r = q.generate(engine, [[5]], Argmax(), max_new_tokens=8, stop_token_ids=[5])[0]
    assert r.token_ids == [5] and r.stop_reason == q.STOP_TOKEN and len(engine.steps) == 1
    # exactly the budget: prompt + max_new_tokens == context is allowed
    r = q.generate(engine, [[1] * 120], Argmax(), max_new_tokens=8)[0]
    assert len(r.token_ids) == 8 and engine.cache.slots.n_free == engine.cache.n_slots


def test_slots_are_given_back_when_a_step_fails():
    class Failing(ScriptedEngine):
        def step(self, entries):
            if len(self.steps) == 2:
                raise RuntimeError("device lost")
            return super().step(entries)

    engine = Failing()
    with pytest.raises(RuntimeError, match="device lost"):
        q.generate(engine, [[1, 2], [3]], Argmax(), max_new_tokens=6)
    assert engine.cache.slots.n_free == engine.cache.n_slots and engine.cache.pages_held() == 0


def test_on_token_sees_every_token_in_order():
    seen = []
    results = q.generate(ScriptedEngine(), [[1, 2], [3]], Argmax(), max_new_tokens=3,
                         on_token=lambda i, t: seen.append((i, t)))
    assert [t for i, t in seen if i == 0] == results[0].token_ids
    assert [t for i, t in seen if i == 1] == results[1].token_ids


def test_sampling_params_follow_the_reference_checks():
    p = q.SamplingParams()
    assert (p.mode, p.temperature, p.top_k, p.top_p, p.seed, p.valid_vocab_size) == ("sample", 0.6, 20, 0.95, 42, 0)
    for bad in ({"temperature": 0.0}, {"temperature": float("inf")}, {"top_k": -1}, {"top_p": 0.0}, {"top_p": 1.5},
                {"mode": "beam"}, {"valid_vocab_size": -1}):
        with pytest.raises(ValueError):
            q.SamplingParams(**bad)
    q.SamplingParams(mode="greedy", temperature=0.0)             # unused options are not checked when greedy
    us = [q.uniform_for(42, s, t) for s in range(4) for t in range(4)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) == 16
    assert q.uniform_for(42, 3, 5) == q.uniform_for(42, 3, 5) != q.uniform_for(43, 3, 5)


class AheadEngine(ScriptedEngine):
    """The scripted engine with the device-token path: a decode step may take its token ids from the
    array the chooser wrote ("on the device") instead of from the entries."""
    device_tokens = True

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.wasted = 0

    def step(self, entries, device_tokens=None):
        if device_tokens is not None:
            assert len(device_tokens) == len(entries) and all(list(e.tokens) == [0] for e in entries)
            entries = [q.StepEntry(e.slot, [int(t)], e.want) for e, t in zip(entries, device_tokens)]
        return super().step(entries)


class AheadArgmax(Argmax):
    class Pending:
        def __init__(self, ids):
            self.device_ids = np.asarray(ids)

        def result(self):
            return [int(t) for t in self.device_ids]

    def choose_async(self, logits, sequence_ids, steps):
        return self.Pending(self.choose(logits, sequence_ids, steps))


def test_running_ahead_gives_the_same_tokens_and_frees_everything():
    prompts = [[1, 2, 3], [7], [4, 4, 4, 4, 4, 4, 4], [9, 9], [5]]
    stops = [28, 22, 5]
    plain_engine, ahead_engine = ScriptedEngine(), AheadEngine()
    want = q.generate(plain_engine, prompts, Argmax(), max_new_tokens=9, stop_token_ids=stops)
    chooser = AheadArgmax()
    got = q.generate(ahead_engine, prompts, chooser, max_new_tokens=9, stop_token_ids=stops)
    assert [(r.token_ids, r.stop_reason) for r in got] == [(r.token_ids, r.stop_reason) for r in want]
    assert ahead_engine.cache.slots.n_free == ahead_engine.cache.n_slots and ahead_engine.cache.pages_held() == 0
    # a sequence that drew a stop token ran at most one step too many, never more
    assert len(plain_engine.steps) <= len(ahead_engine.steps) <= len(plain_engine.steps) + 1
    rows_plain = sum(len(s) for s in plain_engine.steps)
    rows_ahead = sum(len(s) for s in ahead_engine.steps)
    n_stopped = sum(r.stop_reason == q.STOP_TOKEN for r in want)
    assert rows_plain <= rows_ahead <= rows_plain + n_stopped
    # sequences that reach their budget run no extra step; the random streams are numbered as in the plain loop
    assert chooser.calls[0] == ([0, 1, 2, 3, 4], [0] * 5) and chooser.calls[1][1][0] == 1
    again = q.generate(AheadEngine(max_tokens=64 * 2), prompts, AheadArgmax(), max_new_tokens=9, stop_token_ids=stops)
    assert [r.token_ids for r in again] == [r.token_ids for r in want]       # several batches, slots reused


def test_random_workloads_against_the_scripted_rule():
    """Hundreds of random workloads (prompt lengths, budgets, stop sets, cache sizes, slot counts, batch sizes)
    through the loop with the scripted engine: every request gets exactly the tokens and the stop reason the
    rule gives, whatever batches the planner made, and the cache is empty afterwards."""
    rng = np.random.default_rng(123)
    for trial in range(150):
        vocab = int(rng.integers(5, 60))
        n_slots = int(rng.integers(1, 7))
        pages = int(rng.integers(2, 9))
        engine = ScriptedEngine(vocab=vocab, max_tokens=64 * pages, max_seq_len=128, n_slots=n_slots)
        max_new = int(rng.integers(0, 40))
        n = int(rng.integers(0, 12))
        prompts = [[int(t) for t in rng.integers(0, vocab, int(rng.integers(1, 128 - max_new + 1)))] for _ in range(n)]
        stops = [int(s) for s in rng.choice(vocab, size=int(rng.integers(0, 4)), replace=False)]
        batch_size = None if rng.integers(0, 2) else int(rng.integers(1, 5))
        results = q.generate(engine, prompts, Argmax(), max_new_tokens=max_new, stop_token_ids=stops, batch_size=batch_size)
        assert len(results) == n
        # the loop that keeps the device one step ahead of the host decides the same
        ahead = AheadEngine(vocab=vocab, max_tokens=64 * pages, max_seq_len=128, n_slots=n_slots)
        ran_ahead = q.generate(ahead, prompts, AheadArgmax(), max_new_tokens=max_new, stop_token_ids=stops, batch_size=batch_size)
        assert [(r.token_ids, r.stop_reason) for r in ran_ahead] == [(r.token_ids, r.stop_reason) for r in results], trial
        assert ahead.cache.pages_held() == 0 and not ahead.sums
        for prompt, r in zip(prompts, results):
            want, why = expected(prompt, max_new, set(stops), vocab)
            assert (r.token_ids, r.stop_reason) == (want, why), (trial, prompt, max_new, stops)
        assert engine.cache.pages_held() == 0 and not engine.sums
        assert engine.peak_slots <= min(n_slots, batch_size or n_slots)
        # the planner alone: batches are consecutive, respect slots, pages and the batch size, and cover every request
        if n:
            batches = q.plan_batches([len(p) for p in prompts], max_new, pages, n_slots, 64, batch_size)
            assert [i for b in batches for i in b] == list(range(n))
            for b in batches:
                assert len(b) <= min(n_slots, batch_size or n_slots)
                assert sum(-(-(len(prompts[i]) + max_new) // 64) for i in b) <= pages
