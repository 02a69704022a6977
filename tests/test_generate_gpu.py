"""Generation through the Python entry point and the command line, against the plain loop."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import bf16_tolerance, make_folder, plain_logits, random_tokens, tiny
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("gen")
    return {name: make_folder(base, tiny(name), seed=31 + i, name=name) for i, name in enumerate("AB")}


def test_greedy_generation_tiny_a_matches_the_plain_loop(folders):
    """BASELINE's Tiny-A workload: prompts of 5, 17 and 1 tokens together, 8 greedy steps, 32-bit."""
    import qwen3_b200 as q
    folder, weights = folders["A"]
    cfg = tiny("A")
    rng = np.random.default_rng(0)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (5, 17, 1)]
    engine = q.Engine.from_folder(folder, dtype="float32", max_tokens=64 * 3)
    got = q.generate_token_ids(engine, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=8))
    for p, r in zip(prompts, got):
        assert r.token_ids == plain.generate_greedy(cfg, weights, p, 8) and r.stop_reason == q.MAX_NEW_TOKENS
    assert engine.cache.pages_held() == 0
    # a stop token ends its sequence early; the others go on
    stop = got[1].token_ids[2]
    again = q.generate_token_ids(engine, prompts, q.SamplingParams.greedy(),
                                 q.GenerationOptions(max_new_tokens=8, stop_token_ids=[stop]))
    for p, r in zip(prompts, again):
        want = plain.generate_greedy(cfg, weights, p, 8, {stop})
        assert r.token_ids == want
        assert r.stop_reason == (q.STOP_TOKEN if want[-1] == stop else q.MAX_NEW_TOKENS)
    assert again[1].stop_reason == q.STOP_TOKEN and len(again[1].token_ids) <= 3


def test_more_requests_than_slots_run_batch_after_batch(folders):
    import qwen3_b200 as q
    folder, weights = folders["A"]
    cfg = tiny("A")
    rng = np.random.default_rng(1)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (3, 60, 9, 70, 2, 5, 40)]
    engine = q.Engine.from_folder(folder, dtype="float32", max_tokens=64 * 3)       # three pages in all
    got = q.generate_token_ids(engine, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=5))
    for p, r in zip(prompts, got):
        assert r.token_ids == plain.generate_greedy(cfg, weights, p, 5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_tiny_b_follows_the_plain_walk(folders, dtype):
    """BASELINE's Tiny-B workload: prompts of 1, 9, 33 and 64 tokens, 12 steps at temperature 0.7
    with a fixed seed.  Every drawn token is checked against the plain sampling walk over the
    engine's own logits' oracle: in 32-bit the tokens must be the oracle's; in bfloat16 the
    drawn token must be the oracle's draw whenever the draw is not within rounding of a
    boundary, so the sequences are compared through the probability mass instead."""
    import qwen3_b200 as q
    folder, weights = folders["B"]
    cfg = tiny("B")
    rng = np.random.default_rng(2)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (1, 9, 33, 64)]
    params = q.SamplingParams(mode="sample", temperature=0.7, top_k=0, top_p=1.0, seed=1234)
    engine = q.Engine.from_folder(folder, dtype=dtype, max_tokens=64 * 8)
    got = q.generate_token_ids(engine, prompts, params, q.GenerationOptions(max_new_tokens=12))
    again = q.generate_token_ids(engine, prompts, params, q.GenerationOptions(max_new_tokens=12))
    assert [r.token_ids for r in got] == [r.token_ids for r in again]          # same seed, same tokens
    other = q.generate_token_ids(engine, prompts, q.SamplingParams(mode="sample", temperature=0.7, top_k=0,
                                                                    top_p=1.0, seed=99),
                                 q.GenerationOptions(max_new_tokens=12))
    assert [r.token_ids for r in got] != [r.token_ids for r in other]
    # alone or in the batch, a sequence draws the same tokens: its stream is its own
    alone = q.generate_token_ids(engine, [prompts[2]], params, q.GenerationOptions(max_new_tokens=12), sequence_ids=[2])
    if dtype == "float32":
        assert alone[0].token_ids == got[2].token_ids
    else:
        # bfloat16 logits of a row do not depend on the batch either up to 8 rows (one kernel, same order of sums)
        assert alone[0].token_ids == got[2].token_ids
    for i, (p, r) in enumerate(zip(prompts, got)):
        assert len(r.token_ids) == 12
        tokens = list(p)
        for step, t in enumerate(r.token_ids):
            exact = plain_logits(cfg, weights, tokens)[-1]
            u = q.uniform_for(1234, i, step)
            want = plain.sample_row(exact.astype(np.float32), np.float32(0.7), 0, np.float32(1.0), u)
            if dtype == "float32" and t != want:
                # the engine's logits differ from the oracle's in the last bits: accept the neighbour
                # in the sorted order only if the draw sits on the boundary between the two
                probs = np.exp((exact - exact.max()) / 0.7)
                probs /= probs.sum()
                order = np.lexsort((np.arange(len(probs)), -exact))
                cum = np.cumsum(probs[order])
                where = int(np.searchsorted(cum, u, side="right"))
                near = abs(cum[where] - u) < 1e-4 or (where > 0 and abs(cum[where - 1] - u) < 1e-4)
                assert near and t in order[max(where - 1, 0):where + 2], (i, step, t, want)
            if dtype == "bfloat16" and t != want:
                # The engine's logits lie within `tol` of the oracle's (the yardstick of the logits tests).  Under
                # any such change a token surely precedes t in the sorted order if its logit exceeds t's by more
                # than 2 tol, surely follows it if it falls short by more than 2 tol, and every probability changes
                # by at most the factor exp(2 tol / temperature).  The draw has to fall between the least weight
                # that can lie before t and the most that can lie before or on it (a band of a tenth or two of the unit
                # interval on this flat distribution: a wrong stream or walk misses it at most draws).
                tol = bf16_tolerance(cfg, weights, tokens, plain_logits(cfg, weights, tokens))
                probs = np.exp((exact - exact.max()) / 0.7)
                probs /= probs.sum()
                factor = float(np.exp(2.0 * tol / 0.7))
                others = np.arange(len(probs)) != t
                before_least = probs[exact - exact[t] > 2.0 * tol].sum() / factor
                before_most = probs[others & (exact - exact[t] >= -2.0 * tol)].sum() * factor
                assert before_least <= u < before_most + probs[t] * factor, (i, step, t, want, u, before_least, before_most)
            tokens.append(t)


def test_command_line_with_raw_token_ids(folders):
    import qwen3_b200 as q
    folder, weights = folders["A"]
    cfg = tiny("A")
    prompts = [[7, 8, 9], [100, 3]]
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen3_chat"), folder, "--greedy", "--dtype",
                          "float32", "--max-new-tokens", "6", "--max-context", "64", "--tokens", "7,8,9", "--tokens",
                          "100 3", "--stop-token", "255"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.strip().splitlines() if l and l[0].isdigit()]
    assert len(lines) == 2
    stops = {cfg["eos_token_id"], cfg["bos_token_id"], 255}
    for p, line in zip(prompts, lines):
        ids = [int(t) for t in line.split("#")[0].strip().split(",")]
        assert ids == plain.generate_greedy(cfg, weights, p, 6, stops)


def test_chat_loop_with_a_tokenizer(tmp_path):
    """The chat loop end to end on a tiny random model with a tokenizer of its own: template, encoding, generation
    limited to the tokenizer's ids, decoding and the turn handling.  The same message gives the same answer after
    /clear (every turn prefills the whole history into a fresh sequence), an answer cut by --max-new-tokens says
    so (the model's stop ids lie outside the tokenizer's ids here, so no answer ends by itself), and /exit leaves
    with 0."""
    from test_cli import make_tokenizer
    folder, _ = make_folder(tmp_path, tiny("C"), seed=5)
    make_tokenizer(tmp_path)
    os.replace(os.path.join(str(tmp_path), "tokenizer.json"), os.path.join(folder, "tokenizer.json"))
    script = "hello world\n/clear\nhello world\n/think off\nhello\n/help\n/exit\n"
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen3_chat"), folder, "--greedy", "--dtype", "float32",
                          "--max-new-tokens", "4", "--max-context", "128"], input=script, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    turns = out.stdout.split("[the answer was cut at --max-new-tokens]")
    assert len(turns) == 4, out.stdout                           # three answers, each cut after 4 tokens
    first = turns[0].split("> ", 1)[1]
    second = turns[1].split("> > ", 1)[1]                         # the prompts of /clear and of the next message
    assert first == second and first.strip() != ""
    assert "/think on" in out.stdout                              # /help printed the commands
