"""The plain implementation checked against itself and against closed forms, so that the
oracle of the GPU tests is not taken on trust."""
import math

import numpy as np
import pytest

from helpers import make_folder, plain_logits, random_tokens, tiny
from plain import qwen3_plain as plain


def test_round_bf16_matches_torch():
    torch = pytest.importorskip("torch")
    x = np.random.default_rng(0).normal(0, 3, 10000)
    x[:4] = [1.00390625, 1.01171875, -1.00390625, 0.0]          # ties: round to even
    want = torch.tensor(x, dtype=torch.float32).to(torch.bfloat16).double().numpy()
    np.testing.assert_array_equal(plain.round_bf16(x), want)


def test_rms_norm_closed_form():
    x = np.array([[3.0, 4.0, 0.0, 0.0]])
    y = plain.rms_norm(x, np.array([1.0, 2.0, 1.0, 1.0]), 0.75)
    inv = 1.0 / math.sqrt((9 + 16) / 4 + 0.75)
    np.testing.assert_allclose(y, [[3 * inv, 8 * inv, 0, 0]])


def test_rope_is_a_rotation_of_half_split_pairs():
    cos, sin = plain.rope_table(50, 8, 10000.0)
    assert cos.shape == (50, 4) and cos[0].tolist() == [1, 1, 1, 1] and sin[0].tolist() == [0, 0, 0, 0]
    np.testing.assert_allclose(cos[7, 1], math.cos(7 * 10000.0 ** (-2 / 8)), rtol=1e-6)
    x = np.random.default_rng(1).normal(size=(3, 2, 8))
    y = plain.apply_rope(x, np.array([0, 5, 49]), cos, sin)
    np.testing.assert_array_equal(y[0], x[0])
    np.testing.assert_allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-6)
    # pair (i, i + d/2): rotating (1, 0) by the angle gives (cos, sin)
    e = np.zeros((1, 1, 8))
    e[0, 0, 2] = 1.0
    r = plain.apply_rope(e, np.array([5]), cos, sin)[0, 0]
    np.testing.assert_allclose([r[2], r[6]], [cos[5, 2], sin[5, 2]])
    # scores depend on the distance of positions only
    q, k = x[0, 0], x[1, 1]
    def dot(pq, pk):
        a = plain.apply_rope(q[None, None], np.array([pq]), cos, sin)[0, 0]
        b = plain.apply_rope(k[None, None], np.array([pk]), cos, sin)[0, 0]
        return a @ b
    np.testing.assert_allclose(dot(10, 3), dot(40, 33), rtol=1e-5)


def test_attention_is_causal_grouped_and_scaled():
    rng = np.random.default_rng(2)
    T, nq, nkv, d = 6, 4, 2, 8
    q, k, v = rng.normal(size=(T, nq, d)), rng.normal(size=(T, nkv, d)), rng.normal(size=(T, nkv, d))
    out = plain.gqa_attention(q, k, v)
    np.testing.assert_allclose(out[0, :, :], v[0, [0, 0, 1, 1], :])       # position 0 sees itself only
    k2, v2 = k.copy(), v.copy()
    k2[4:], v2[4:] = 9.0, -9.0
    np.testing.assert_array_equal(plain.gqa_attention(q, k2, v2)[:4], out[:4])   # later keys change nothing
    s = (k[:3, 1] @ q[2, 3]) / math.sqrt(d)
    w = np.exp(s - s.max())
    np.testing.assert_allclose(out[2, 3], (w / w.sum()) @ v[:3, 1])
    win = plain.gqa_attention(q, k, v, window=2)
    s = (k[4:6, 0] @ q[5, 0]) / math.sqrt(d)
    w = np.exp(s - s.max())
    np.testing.assert_allclose(win[5, 0], (w / w.sum()) @ v[4:6, 0])


def test_silu_and_embedding():
    np.testing.assert_allclose(plain.silu_multiply(np.array([0.0, 1.0]), np.array([5.0, 2.0])),
                               [0.0, 2.0 / (1 + math.exp(-1))])
    table = np.arange(12.0).reshape(4, 3)
    np.testing.assert_array_equal(plain.embedding([2, 9, -1, 0], table), [[6, 7, 8], [0, 0, 0], [0, 0, 0], [0, 1, 2]])


@pytest.mark.parametrize("name", ["A", "B"])
def test_forward_is_causal_and_uses_tied_or_untied_head(tmp_path, name):
    cfg = tiny(name)
    _, w = make_folder(tmp_path, cfg, seed=4)
    rng = np.random.default_rng(3)
    toks = random_tokens(rng, 12, cfg["vocab_size"])
    full = plain_logits(cfg, w, toks)
    assert full.shape == (12, cfg["vocab_size"]) and np.all(np.isfinite(full))
    np.testing.assert_allclose(plain_logits(cfg, w, toks[:7]), full[:7], atol=1e-12)
    changed = toks[:]
    changed[9] = (changed[9] + 1) % cfg["vocab_size"]
    again = plain_logits(cfg, w, changed)
    np.testing.assert_allclose(again[:9], full[:9], atol=1e-12)
    assert np.max(np.abs(again[9:] - full[9:])) > 1e-6
    assert ("lm_head.weight" in w) == (not cfg["tie_word_embeddings"])


def test_sample_row_follows_the_reference_rules():
    logits = np.array([2.0, 2.0, 1.0, -10.0])
    # top_k = 3 keeps ids 0, 1, 2; top_p = 0.8: weights 1, 1, e^-1 -> 0.8 * 2.37 = 1.89 <= 2 -> ids 0 and 1 only
    draws = {plain.sample_row(logits, 1.0, 3, 0.8, u) for u in np.linspace(0, 0.999999, 101)}
    assert draws == {0, 1}
    assert plain.sample_row(logits, 1.0, 3, 0.8, 0.49) == 0 and plain.sample_row(logits, 1.0, 3, 0.8, 0.51) == 1
    # top_k = 1 with a tie keeps both equals (every score that reaches the k-th best stays)
    assert {plain.sample_row(logits, 1.0, 1, 1.0, u) for u in (0.1, 0.9)} == {0, 1}
    assert plain.sample_row(np.array([0.0, 5.0, 1.0]), 0.5, 1, 1.0, 0.7) == 1
    # the valid prefix hides later ids
    assert {plain.sample_row(np.array([0.0, 1.0, 50.0]), 1.0, 0, 1.0, u, valid=2) for u in (0.0, 0.5, 0.99)} == {0, 1}
    with pytest.raises(RuntimeError):
        plain.sample_row(np.array([0.0, np.nan]), 1.0, 0, 1.0, 0.5)
    assert plain.argmax_lowest(np.array([1.0, 3.0, 3.0, np.nan])) == 1


def test_generate_greedy_keeps_the_stop_token_and_stops(tmp_path):
    cfg = tiny("A")
    _, w = make_folder(tmp_path, cfg, seed=4)
    out = plain.generate_greedy(cfg, w, [5, 6, 7], 6)
    assert len(out) == 6
    stopped = plain.generate_greedy(cfg, w, [5, 6, 7], 6, stop_token_ids={out[2]})
    first = out.index(out[2])
    assert stopped == out[:first + 1]
