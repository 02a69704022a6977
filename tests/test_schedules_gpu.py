"""Schedules that a real batch takes and the plain cuttings do not reach: decode steps whose
number of live sequences is no captured batch size (padding rows), batches that shrink across
those sizes, prompts continued by several tokens at a position above 0, steps that mix such
continuations with sequences going on by one token, replayed steps against freshly launched
ones, token ids read on the device, and the widths of the 8B shape through the engine (so that
the kernels of the measured prompt step produce checked logits)."""
import numpy as np
import pytest

import schedules
from helpers import FP32_TOL, bf16_tolerance, make_folder, plain_logits, random_tokens, tiny
from plain import qwen3_plain as plain
from test_engine_gpu import check, make_requests, run_steps

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {name: make_folder(base, tiny(name), seed=31 + i, name=name) for i, name in enumerate("ABCD")}


def engine_for(folder, dtype, max_tokens, **kw):
    from qwen3_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


# live sequences per decode step: 70 and 66 pad to 96 rows, 65 too, 64 is exact, 33 pads to 40, 20 to 24,
# 17 to 24, 16 exact, 13 and 9 pad to 16, 8 and below are exact
LIVE = [70, 66, 65, 64, 33, 20, 17, 16, 13, 9, 8, 5, 1]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_decode_steps_with_padding_rows(folders, name, dtype):
    """A batch of 70 whose sequences end at different steps, so that the captured decode step runs with
    padding rows (70 of 96, 33 of 40, 13 of 16, 9 of 16 ...) and shrinks across the captured sizes."""
    from qwen3_b200.engine.engine import decode_bucket
    assert [decode_bucket(n) for n in (70, 65, 64, 33, 20, 13, 9, 8)] == [96, 96, 64, 40, 24, 16, 16, 8]
    folder, weights = folders[name]
    cfg = tiny(name)
    totals, prompts = schedules.shrinking(LIVE)
    requests = make_requests(cfg, totals, seed=7)
    prompt_lengths = dict(zip(requests, prompts))
    steps, rows = schedules.batched(requests, prompt_lengths, len(totals))
    assert [len(s["entries"]) for s in steps[1:]] == LIVE
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, cfg, weights, dtype, "padded decode steps")
    assert sorted(engine._graphs) == [1, 5, 8, 16, 24, 40, 64, 96]
    assert engine.cache.pages_held() == 0 and engine.cache.slots.n_free == engine.cache.n_slots
    # the same batch once more in the same engine: the captured steps are replayed with other slots and pages
    again = run_steps(engine, steps, rows)
    for key, row in got.items():
        assert np.array_equal(row, again[key]), key


@pytest.mark.parametrize("dtype", DTYPES)
def test_replayed_steps_equal_launched_steps(folders, dtype):
    """The same schedule with captured decode steps and with every step launched afresh: in 32-bit the
    logits are equal bit for bit (a row's sums do not depend on the rows beside it, padding included);
    in bfloat16 they are equal wherever the step has the same number of rows in both engines and
    within the rounding yardstick elsewhere (the product for 9 and more rows splits K by the row count)."""
    folder, weights = folders["B"]
    cfg = tiny("B")
    totals, prompts = schedules.shrinking([13, 9, 8, 3, 3, 1], prompt_of=lambda i: 1 + 7 * (i % 4))
    requests = make_requests(cfg, totals, seed=9)
    steps, rows = schedules.batched(requests, dict(zip(requests, prompts)), len(totals))
    captured = run_steps(engine_for(folder, dtype, schedules.peak_tokens(steps)), steps, rows)
    launched_engine = engine_for(folder, dtype, schedules.peak_tokens(steps), use_graphs=False)
    launched = run_steps(launched_engine, steps, rows)
    assert not launched_engine._graphs
    exact_rows = set()
    for step, out in zip(steps[1:], rows[1:]):
        if len(step["entries"]) <= 8:
            exact_rows.update(out)
    for rid, toks in requests.items():
        tol = bf16_tolerance(cfg, weights, toks, plain_logits(cfg, weights, toks))
        for p in range(len(toks)):
            if (rid, p) not in captured:
                continue
            a, b = captured[(rid, p)], launched[(rid, p)]
            if dtype == "float32" or (rid, p) in exact_rows:
                assert np.array_equal(a, b), (rid, p, float(np.max(np.abs(a - b))))
            else:
                assert np.max(np.abs(a - b)) <= tol, (rid, p)
    check(launched, requests, cfg, weights, dtype, "launched steps")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,cuts", [
    ("B", [200, 66], [[7, 64, 65], [33]]),
    ("C", [300, 131], [[100, 101, 228], [64, 128]]),
    ("D", [300, 333], [[130], [129, 260]]),          # head size 64: continued chunks of 128 and more tokens
])
def test_prompts_continued_by_several_tokens(folders, name, lengths, cuts, dtype):
    folder, weights = folders[name]
    cfg = tiny(name)
    requests = make_requests(cfg, lengths, seed=10)
    steps, rows = schedules.chunked(requests, dict(zip(requests, cuts)))
    assert any(len(s["entries"][0]["tokens"]) > 1 for s in steps[1:])
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == sum(lengths)
    check(got, requests, cfg, weights, dtype, "continued prompts")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,first,chunk", [
    ("A", [90, 30, 64, 12], [40, 5, 64, 1], [17, 1, 1, 1]),
    ("D", [420, 40, 200, 10, 129], [100, 5, 64, 1, 128], [150, 1, 3, 1, 1]),
])
def test_steps_that_mix_continuations_with_single_tokens(folders, name, lengths, first, chunk, dtype):
    folder, weights = folders[name]
    cfg = tiny(name)
    requests = make_requests(cfg, lengths, seed=12)
    steps, rows = schedules.mixed(requests, dict(zip(requests, first)), dict(zip(requests, chunk)))
    sizes = [sorted({len(e["tokens"]) for e in s["entries"]}) for s in steps[1:]]
    assert any(len(s) > 1 and s[0] == 1 for s in sizes), "no step mixes one token with several"
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == sum(lengths)
    check(got, requests, cfg, weights, dtype, "mixed steps")
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("use_graphs", [True, False])
def test_token_ids_read_on_the_device(folders, dtype, use_graphs):
    """A decode step that reads its ids from a device tensor gives the logits of the step that was
    handed the same ids from the host, bit for bit."""
    import torch
    from qwen3_b200 import StepEntry
    folder, _ = folders["B"]
    cfg = tiny("B")
    rng = np.random.default_rng(13)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (9, 1, 33)]
    nxt = random_tokens(rng, 3, cfg["vocab_size"])
    outs = []
    for on_device in (False, True):
        engine = engine_for(folder, dtype, 64 * 3, use_graphs=use_graphs)
        slots = [engine.new_sequence() for _ in prompts]
        engine.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
        if on_device:
            ids = torch.tensor(nxt, dtype=torch.int32, device=engine.device)
            logits = engine.step([StepEntry(s, [0], [0]) for s in slots], device_tokens=ids)
        else:
            logits = engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt)])
        outs.append(logits.cpu().numpy().copy())
    assert np.array_equal(outs[0], outs[1])


# ---------------------------------------------------------------------------- the widths of the 8B shape
WIDE = dict(tiny("B"), num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
            head_dim=128, intermediate_size=12288, vocab_size=151936, max_position_embeddings=4096,
            bos_token_id=151643, eos_token_id=151645, rms_norm_eps=1e-6, torch_dtype="bfloat16")
WIDE_PROMPTS = [300, 129, 700, 5]
WIDE_DECODED = 3


@pytest.fixture(scope="module")
def wide():
    """Two layers of the 8B widths with random weights; exact and bfloat16-emulated logits of the plain model
    at the rows the test asks for (the last prompt position and every decoded one)."""
    import torch
    import qwen3_b200 as q
    config = q.config_from_dict(WIDE)
    model = q.build_model(config.plan())
    tensors = q.random_weights(model.weight_specs(), seed=5, dtype=torch.bfloat16, device="cuda")
    weights = {}
    for k, v in tensors.items():
        big = v.numel() > 100_000_000 and "embed" in k                   # the embedding is only gathered from
        weights[k] = v.float().cpu().numpy() if big else v.double().cpu().numpy()
    rng = np.random.default_rng(14)
    requests = {f"w{i}": random_tokens(rng, n + WIDE_DECODED, WIDE["vocab_size"]) for i, n in enumerate(WIDE_PROMPTS)}
    wanted = {rid: list(range(n - 1, n + WIDE_DECODED)) for rid, n in zip(requests, WIDE_PROMPTS)}
    exact = {rid: plain.forward(WIDE, weights, toks, rows=wanted[rid]) for rid, toks in requests.items()}
    emulated = {rid: plain.forward(WIDE, weights, toks, rnd=plain.round_bf16, rnd_logits=plain.identity, rows=wanted[rid])
                for rid, toks in requests.items()}
    host = {k: v.cpu() for k, v in tensors.items()}
    del tensors
    torch.cuda.empty_cache()
    return config, host, requests, wanted, exact, emulated


@pytest.mark.parametrize("dtype", DTYPES)
def test_8b_widths_in_unequal_batches(wide, dtype, monkeypatch):
    """Prompts of 300, 129, 700 and 5 tokens in batches of two with two slots (the second batch takes the
    slots and pages of the first), three tokens decoded each: 32-bit within 1e-4 of the float64 model,
    bfloat16 within its rounding yardstick.  In bfloat16 the step of 705 tokens runs the product on pairs
    of SMs (its gated form too) and the tcgen05 attention at head size 128 with 32:8 heads."""
    import torch
    import qwen3_b200 as q
    from qwen3_b200.csrc import ops
    from qwen3_b200.engine.engine import Engine
    config, host, requests, wanted, exact, emulated = wide
    calls = {"pair": 0, "pair_gated": 0, "pair_qkv": 0, "attention_tc": 0, "skinny": 0, "decode_attention": 0}
    real_pair, real_tc, real_skinny, real_dec = ops.gemm_tcgen05_pair, ops.attention_prefill_tc, ops.gemm_skinny, ops.attention_decode_fused
    real_qkv = ops.gemm_tcgen05_pair_qkv

    def pair_qkv(*a, **k):
        calls["pair_qkv"] += 1
        return real_qkv(*a, **k)

    def pair(x, w, out, gated=False, splits=1):
        calls["pair_gated" if gated else "pair"] += 1
        return real_pair(x, w, out, gated, splits)

    def tc(*a, **k):
        calls["attention_tc"] += 1
        return real_tc(*a, **k)

    def skinny(*a, **k):
        calls["skinny"] += 1
        return real_skinny(*a, **k)

    def dec(*a, **k):
        calls["decode_attention"] += 1
        return real_dec(*a, **k)

    monkeypatch.setattr(ops, "gemm_tcgen05_pair", pair)
    monkeypatch.setattr(ops, "gemm_tcgen05_pair_qkv", pair_qkv)
    from qwen3_b200.parts import attention as attention_part
    monkeypatch.setattr(attention_part, "fused_projection_rows", 256)      # the prompts here are hundreds of tokens long
    monkeypatch.setattr(ops, "attention_prefill_tc", tc)
    monkeypatch.setattr(ops, "gemm_skinny", skinny)
    monkeypatch.setattr(ops, "attention_decode_fused", dec)
    model = q.build_model(config.plan())
    model.bind({k: v.cuda() for k, v in host.items()}, torch.float32 if dtype == "float32" else torch.bfloat16, "cuda")
    prompt_lengths = dict(zip(requests, WIDE_PROMPTS))
    steps, rows = schedules.batched(requests, prompt_lengths, 2)
    engine = Engine(model, config, max_tokens=schedules.peak_tokens(steps), max_seq_len=1024, n_slots=2)
    got = run_steps(engine, steps, rows)
    assert engine.cache.pages_held() == 0
    engine.check_kernels()
    for rid in requests:
        assert float(np.abs(exact[rid]).max()) > 0.5
        tol = FP32_TOL if dtype == "float32" else 4.0 * float(np.max(np.abs(emulated[rid] - exact[rid]))) + 1e-6
        for i, p in enumerate(wanted[rid]):
            err = float(np.max(np.abs(got[(rid, p)] - exact[rid][i])))
            assert err <= tol, f"[{dtype}] request {rid} position {p}: max abs err {err:.3e} > {tol:.3e}"
    if dtype == "bfloat16":
        # 705 tokens: every projection on pairs of SMs, q/k/v with norm, rotation and cache write in its epilogue
        assert calls["pair"] >= 2 * 2 and calls["pair_gated"] >= 2 * 2 and calls["pair_qkv"] >= 2, calls
        assert calls["attention_tc"] == 2 * 2 and calls["decode_attention"] > 0 and calls["skinny"] > 0, calls
    del engine, model
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_few_sequences_growing_past_the_long_context_bound(folders, name, dtype, monkeypatch):
    """One sequence, then two of unequal lengths, decoded token by token from below the bound at which the engine
    captures steps of a few sequences apart (lowered to 200 tokens here) to beyond it: the logits agree with the
    plain model on both sides of the bound and at the step that crosses it, both sets of captured steps were used,
    and in bfloat16 the one-launch attention ran with clusters beyond the portable size (more than eight key
    splits per sequence and kv head, some of them without a page)."""
    from qwen3_b200.csrc import ops
    from qwen3_b200.engine import engine as engine_module
    from qwen3_b200.parts import attention as attention_part
    monkeypatch.setattr(engine_module, "LONG_CONTEXT", 200)
    monkeypatch.setattr(attention_part, "long_context_keys", 200)
    splits_seen = set()
    real = ops.attention_decode_fused

    def fused(*a, **k):
        splits_seen.add(a[18] if len(a) > 18 else k.get("n_splits"))
        return real(*a, **k)
    monkeypatch.setattr(ops, "attention_decode_fused", fused)
    folder, weights = folders[name]
    cfg = tiny(name)
    for lengths, prompts in (([230], {"r0": 180}), ([215, 240], {"r0": 190, "r1": 170})):
        requests = make_requests(cfg, lengths, seed=len(lengths))
        steps, rows = schedules.batched(requests, prompts, len(lengths))
        engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
        got = run_steps(engine, steps, rows)
        check(got, requests, cfg, weights, dtype, f"{len(lengths)} sequences across the bound")
        assert engine._graphs and engine._long_graphs, (list(engine._graphs), list(engine._long_graphs))
        engine.check_kernels()
    if dtype == "bfloat16":
        assert max(splits_seen) > 8 and 8 in splits_seen, splits_seen
