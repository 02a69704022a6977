"""The engine against the plain implementation, in 32-bit and in bfloat16, under every
way of cutting the same requests into steps: whole; the last 32 tokens one by one;
batches of unequal lengths whose shorter requests end earlier, one batch after another
so that slots and pages are used again; long decoding; the first tokens of a sequence."""
import numpy as np
import pytest

import schedules
from helpers import FP32_TOL, bf16_tolerance, make_folder, plain_logits, random_tokens, tiny
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def run_steps(engine, steps, rows):
    """Drive `engine.step` with trace-format steps; returns {(request id, position): logits row}."""
    from qwen3_b200 import StepEntry
    slots, got = {}, {}
    for step, out in zip(steps, rows):
        entries = []
        for e in step["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = engine.new_sequence()
            entries.append(StepEntry(slots[e["id"]], e["tokens"], e["want"]))
        logits = engine.step(entries)
        if out:
            block = logits.cpu().numpy()
            assert block.shape[0] == len(out)
            for key, row in zip(out, block):
                got[key] = row.copy()
        else:
            assert logits is None
        for rid in step["end"]:
            engine.release(slots.pop(rid))
    assert not slots
    return got


def check(got, requests, cfg, weights, dtype, label):
    worst = 0.0
    for rid, toks in requests.items():
        exact = plain_logits(cfg, weights, toks)
        tol = FP32_TOL if dtype == "float32" else bf16_tolerance(cfg, weights, toks, exact)
        for p in range(len(toks)):
            if (rid, p) not in got:
                continue
            err = float(np.max(np.abs(got[(rid, p)] - exact[p])))
            worst = max(worst, err)
            assert np.all(np.isfinite(got[(rid, p)])), f"{label}: request {rid} position {p}: non-finite logits"
            assert err <= tol, (f"{label} [{dtype}]: request {rid} position {p} of {len(toks)}: "
                                f"max abs err {err:.3e} > {tol:.3e}")
    return worst


def make_requests(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": random_tokens(rng, n, cfg["vocab_size"]) for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {name: make_folder(base, tiny(name), seed=11 + i, name=name) for i, name in enumerate("ABCD")}


def engine_for(folder, dtype, max_tokens):
    from qwen3_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("A", [5, 17, 1, 64, 65, 100]), ("B", [1, 9, 33, 64, 130]),
                                          ("C", [2, 63, 129, 300]), ("D", [7, 128, 200, 333])])
def test_whole_requests(folders, name, lengths, dtype):
    folder, weights = folders[name]
    cfg = tiny(name)
    requests = make_requests(cfg, lengths, seed=1)
    steps, rows = schedules.whole(requests)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == sum(lengths)
    check(got, requests, cfg, weights, dtype, "whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("A", [5, 40, 100]), ("B", [33, 64, 97, 200]), ("C", [31, 32, 33, 257])])
def test_last_32_tokens_one_by_one(folders, name, lengths, dtype):
    folder, weights = folders[name]
    cfg = tiny(name)
    requests = make_requests(cfg, lengths, seed=2)
    steps, rows = schedules.tail_one_by_one(requests, 32)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, cfg, weights, dtype, "tail one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,prompts,batch", [
    ("A", [13, 25, 9, 70, 66, 20, 128, 3], [5, 17, 1, 64, 65, 12, 100, 3], 3),
    ("B", [13, 21, 45, 76, 30, 200, 65], [1, 9, 33, 64, 30, 129, 2], 4),
    ("C", [200, 90, 300, 64, 150], [100, 63, 257, 1, 64], 2),
    ("D", [300, 140, 9, 260, 131], [129, 128, 1, 256, 130], 3),
])
def test_unequal_batches_one_after_another(folders, name, lengths, prompts, batch, dtype):
    folder, weights = folders[name]
    cfg = tiny(name)
    requests = make_requests(cfg, lengths, seed=3)
    prompt_lengths = {rid: p for rid, p in zip(requests, prompts)}
    steps, rows = schedules.batched(requests, prompt_lengths, batch, want_all_prompt=True)
    # the cache holds exactly what the largest batch needs: later batches reuse slots and pages
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == sum(lengths)
    check(got, requests, cfg, weights, dtype, "unequal batches")
    assert engine.cache.pages_held() == 0 and engine.cache.slots.n_free == engine.cache.n_slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype):
    """One sequence decoded token by token from its first token, across many page edges."""
    folder, weights = folders["C"]
    cfg = tiny("C")
    requests = make_requests(cfg, [400], seed=4)
    steps, rows = schedules.tail_one_by_one(requests, 400)
    engine = engine_for(folder, dtype, 448)
    got = run_steps(engine, steps, rows)
    assert len(got) == 400
    check(got, requests, cfg, weights, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(folders, name, dtype):
    """Sequences of one, two and three tokens, alone and together, whole and token by token."""
    folder, weights = folders[name]
    cfg = tiny(name)
    requests = make_requests(cfg, [1, 2, 3], seed=5)
    engine = engine_for(folder, dtype, 64 * 3)
    for builder in (schedules.whole, lambda r: schedules.tail_one_by_one(r, 32),
                    lambda r: schedules.batched(r, {k: 1 for k in r}, 3)):
        steps, rows = builder(requests)
        got = run_steps(engine, steps, rows)
        check(got, requests, cfg, weights, dtype, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_does_not_change_logits_beyond_rounding(folders, dtype):
    """The same positions under three cuttings agree with each other much more closely than
    with the exact model in bfloat16, and to rounding in 32-bit."""
    folder, weights = folders["B"]
    cfg = tiny("B")
    requests = make_requests(cfg, [70, 33, 120], seed=6)
    engine = engine_for(folder, dtype, 64 * 6)
    a = run_steps(engine, *schedules.whole(requests))
    b = run_steps(engine, *schedules.tail_one_by_one(requests, 32))
    c = run_steps(engine, *schedules.batched(requests, {"r0": 10, "r1": 33, "r2": 64}, 3))
    for rid, toks in requests.items():
        # 32-bit: different summation orders only; bfloat16: the yardstick of the comparison with the exact model
        tol = 2e-5 if dtype == "float32" else bf16_tolerance(cfg, weights, toks, plain_logits(cfg, weights, toks))
        for other in (b, c):
            for (r, p), row in other.items():
                if r == rid:
                    assert np.max(np.abs(a[(r, p)] - row)) <= tol, (r, p)


def test_checkpoint_stored_in_32_bit_runs_in_both_types(tmp_path):
    """A folder of float32 tensors: exact in the 32-bit engine; the bfloat16 engine rounds the matrices
    (and says so) and then agrees with the plain model of the rounded weights."""
    import qwen3_b200 as q
    cfg = tiny("D")
    folder, weights = make_folder(tmp_path, cfg, seed=77, storage="float32")
    requests = make_requests(cfg, [40, 150], seed=8)
    steps, rows = schedules.tail_one_by_one(requests, 8)
    got = run_steps(engine_for(folder, "float32", schedules.peak_tokens(steps)), steps, rows)
    check(got, requests, dict(cfg, torch_dtype="float32"), weights, "float32", "32-bit storage")
    rounded = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in weights.items()}
    got = run_steps(engine_for(folder, "bfloat16", schedules.peak_tokens(steps)), steps, rows)
    check(got, requests, cfg, rounded, "bfloat16", "32-bit storage, bfloat16 engine")


def test_step_errors_leave_the_cache_unchanged(folders):
    from qwen3_b200 import CacheFull, StepEntry, StepError
    folder, _ = folders["A"]
    engine = engine_for(folder, "float32", 128)
    s = engine.new_sequence()
    with pytest.raises(StepError):
        engine.step([StepEntry(s, [], [])])
    with pytest.raises(StepError):
        engine.step([StepEntry(s, [256], [0])])
    with pytest.raises(StepError):
        engine.step([StepEntry(s, [1, 2], [2])])
    with pytest.raises(CacheFull):
        engine.step([StepEntry(s, list(range(129)), [])])
    assert engine.length(s) == 0 and engine.cache.pages_held() == 0
    assert engine.step([StepEntry(s, [1, 2, 3], [])]) is None
    assert engine.length(s) == 3
    # a failure after the pages were reserved (a kernel that refuses its sizes, memory that runs out while the
    # scratch grows): the pages go back, the length stays, and the same step then runs
    held, real_forward = engine.cache.pages_held(), engine.model.forward

    def failing(ctx, cache):
        raise RuntimeError("launch failed")

    engine.model.forward = failing
    with pytest.raises(RuntimeError, match="launch failed"):
        engine.step([StepEntry(s, list(range(70)), [69])])
    engine.model.forward = real_forward
    assert engine.length(s) == 3 and engine.cache.pages_held() == held
    assert engine.step([StepEntry(s, list(range(70)), [69])]).shape == (1, 256)
    assert engine.length(s) == 73 and engine.cache.pages_held() == 2
    engine.release(s)
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_guard_zones_and_cache_canaries_survive_every_kind_of_step(folders, name, dtype):
    """Every activation buffer lies between guard zones and every cell of the cache starts as a canary.  After
    whole prompts of unequal lengths, a prompt in two chunks, captured decode steps (a padded batch among them,
    whose padding rows write to the spare page) and launched decode steps, the guard zones are intact, exactly the
    cells of the live sequences' tokens were written, and everything else in the cache - free pages, the rows
    behind a sequence's last token - still holds the canary."""
    import torch
    from qwen3_b200 import Engine, StepEntry
    from qwen3_b200.cache import PAGE_TOKENS
    folder, _ = folders[name]
    cfg = tiny(name)
    rng = np.random.default_rng(5)
    canary = 12352.0                                           # a value bfloat16 holds exactly
    for use_graphs in (True, False):
        engine = Engine.from_folder(folder, dtype=dtype, max_tokens=12 * 128, use_graphs=use_graphs, guard_scratch=True)
        for store in engine.cache.stores:
            store.fill_(canary)
        lengths = [70, 5, 64, 1, 33, 100, 65, 9, 17]          # nine live sequences: the captured batch is padded to 16
        slots = [engine.new_sequence() for _ in lengths]
        tokens = [random_tokens(rng, n, cfg["vocab_size"]) for n in lengths]
        engine.step([StepEntry(s, t, [len(t) - 1]) for s, t in zip(slots[:4], tokens[:4])])
        engine.step([StepEntry(s, t[:len(t) // 2], []) for s, t in zip(slots[4:], tokens[4:])])          # a prompt in two
        engine.step([StepEntry(s, t[len(t) // 2:], [0]) for s, t in zip(slots[4:], tokens[4:])])         # chunks
        for _ in range(3):
            engine.step([StepEntry(s, [int(rng.integers(0, cfg["vocab_size"]))], [0]) for s in slots])
        released_pages = {p for g in engine.cache.groups for p in g.held_pages(slots[-1])}
        engine.release(slots.pop())                             # eight left: a batch that needs no padding
        engine.step([StepEntry(s, [int(rng.integers(0, cfg["vocab_size"]))], [0]) for s in slots])
        torch.cuda.synchronize()
        assert engine.scratch_violations() == []
        assert (len(engine._graphs) > 0) == use_graphs
        for group, store in zip(engine.cache.groups, engine.cache.stores):
            written = torch.zeros(store.shape[2], PAGE_TOKENS, dtype=torch.bool)
            for s in slots:
                pages, n = group.held_pages(s), engine.cache.length(s)
                assert len(pages) == -(-n // PAGE_TOKENS)
                for p in range(n):
                    written[pages[p // PAGE_TOKENS], p % PAGE_TOKENS] = True
            # [layers, keys/values, page, head, row, d] -> touched [page, row]: any cell that differs from the canary
            touched = (store != canary).any(dim=-1).any(dim=3).any(dim=1).any(dim=0).cpu()
            every = (store != canary).any(dim=-1).all(dim=3).all(dim=1).all(dim=0).cpu()
            spare = store.shape[2] - 1
            released = touched.clone()
            released[:spare] &= ~written[:spare]
            # the released sequence's pages keep its rows; apart from them nothing outside the live tokens is touched
            live_pages = {p for s in slots for p in group.held_pages(s)}
            stray = [(int(p), int(r)) for p, r in released[:spare].nonzero() if int(p) in live_pages]
            assert stray == [], f"cells behind a sequence's last token were written: {stray[:5]}"
            assert bool(every[:spare][written[:spare]].all()), "a live token's keys or values were not written in some layer or head"
            free_touched = {int(p) for p, _ in released[:spare].nonzero()} - live_pages
            assert free_touched <= released_pages, free_touched          # only the released sequence's own page


def test_8b_layer_shapes_in_32_bit_match_the_plain_model():
    """One layer of the Qwen3-8B shape (hidden 4096, 32/8 heads of 128, intermediate 12288, vocabulary
    151936) in true 32-bit: whole, cut in two, and token by token agree with the float64 plain model to
    1e-4.  TF32 or bfloat16 anywhere on the path would miss this bound by orders of magnitude."""
    import torch
    import qwen3_b200 as q
    cfg = dict(tiny("B"), num_hidden_layers=1, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
               head_dim=128, intermediate_size=12288, vocab_size=151936, max_position_embeddings=4096,
               bos_token_id=151643, eos_token_id=151645, torch_dtype="bfloat16")
    config = q.config_from_dict(cfg)
    model = q.build_model(config.plan())
    tensors = q.random_weights(model.weight_specs(), seed=8, dtype=torch.bfloat16, device="cuda")
    weights = {k: v.double().cpu().numpy() for k, v in tensors.items()}
    model.bind(tensors, torch.float32, "cuda")
    from qwen3_b200.engine.engine import Engine
    engine = Engine(model, config, max_tokens=128, max_seq_len=128)
    rng = np.random.default_rng(3)
    toks = random_tokens(rng, 9, cfg["vocab_size"])
    exact = plain_logits(cfg, weights, toks)
    requests = {"r": toks}
    whole = run_steps(engine, *schedules.whole(requests))
    one = run_steps(engine, *schedules.tail_one_by_one(requests, 4))
    for p in range(len(toks)):
        assert np.max(np.abs(whole[("r", p)] - exact[p])) <= FP32_TOL, p
        if ("r", p) in one:
            assert np.max(np.abs(one[("r", p)] - exact[p])) <= FP32_TOL, p
    assert float(np.abs(exact).max()) > 0.5      # the bound is meaningful: logits are of order one
