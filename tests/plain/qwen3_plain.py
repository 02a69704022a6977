"""Plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

This file is the oracle of the test suite.  It shares no code with the product
package: it takes a plain dict (the keys of config.json) and a dict of NumPy
arrays keyed by checkpoint tensor name, and it recomputes every position of a
sequence from scratch.

The reference's model code cannot be compiled or imported on a CPU-only
machine (its `qwen3/core` headers are absent from the checkout and every model
file needs CUDA and cuBLAS), so the numerics here rest on the formulas of the
reference's sources, each cited as file:line of RicardoMin/Qwen3-Runtime-ByYourself.
Only the configuration parser of the reference compiles on the CPU; it anchors
`tests/golden/`.

`rnd` is a rounding hook: the identity gives the exact (float64) model; passing
`round_bf16` reproduces the reference's bfloat16 rounding points, which is how
the tests size the tolerance of the bfloat16 engine.
"""
from __future__ import annotations

import math

import numpy as np


def identity(x):
    return x


def round_bf16(x):
    """Round-to-nearest-even to bfloat16, returned in float64."""
    f = np.asarray(x, dtype=np.float32)
    bits = f.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32).astype(np.float64)
    return out.reshape(np.shape(x))


# ----------------------------------------------------------------------------- parts


def embedding(token_ids, table):
    """x[t,:] = E[id[t],:]; an id outside the table gives a zero row.
    src/ops/embedding.cu:38-52"""
    ids = np.asarray(token_ids, dtype=np.int64)
    out = np.zeros((ids.shape[0], table.shape[1]), dtype=np.float64)
    ok = (ids >= 0) & (ids < table.shape[0])
    out[ok] = table[ids[ok]]
    return out


def rms_norm(x, weight, eps, rnd=identity):
    """inv = rsqrt(mean(x^2) + eps); y = rnd(rnd(x*inv) * w).  The epsilon is
    added to the mean inside the root; the weight multiplies directly (no 1+w).
    src/ops/rms_norm.cu:87-120"""
    x = np.asarray(x, dtype=np.float64)
    inv = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return rnd(rnd(x * inv) * weight)


def linear(x, w, rnd=identity):
    """y = x . W^T with W stored [out, in]; no bias.  src/ops/linear.cpp:165-193"""
    return rnd(np.asarray(x, dtype=np.float64) @ np.asarray(w, dtype=np.float64).T)


def rope_table(n_positions, head_dim, theta):
    """inv_freq_i = theta^(-2i/d); angle = pos * inv_freq_i in float64; the
    cosine and sine are stored as float32.  src/ops/rope.cu:276-295"""
    half = head_dim // 2
    inv_freq = np.array([math.pow(float(theta), -(2.0 * i) / head_dim) for i in range(half)])
    angle = np.arange(n_positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    cos = np.cos(angle).astype(np.float32).astype(np.float64)
    sin = np.sin(angle).astype(np.float32).astype(np.float64)
    return cos, sin


def apply_rope(x, positions, cos, sin, rnd=identity):
    """Half-split rotation of the pairs (i, i+d/2) of every head.
    x: [T, heads, d].  src/ops/rope.cu:60-84
    Tables narrower than d/2 (not a Qwen3 option: the reference rotates the whole head; it exists for the
    tests of the rotation kernels alone) rotate only the first 2 * width values, in pairs (i, i + width),
    and leave the rest as they are."""
    half = cos.shape[-1]
    c = cos[positions][:, None, :]
    s = sin[positions][:, None, :]
    first, second, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return rnd(np.concatenate([first * c - second * s, second * c + first * s, rest], axis=-1))


def gqa_attention(q, k, v, rnd=identity, window=None):
    """Causal grouped-query attention of one whole sequence.
    q: [T, nq, d]; k, v: [T, nkv, d].  Query head h reads kv head h // (nq/nkv)
    (src/ops/gqa_attention.cu:42-44); a query at position p sees keys 0..p by the
    loop bound (:84-86); score = dot * d^-0.5 with the scale after the dot (:117,
    :326); softmax and the weighted sum are exact here where the kernel runs an
    online softmax in 32-bit (:119-144); out = sum / normaliser (:152-153).
    `window` (not a Qwen3 dense option: the reference rejects it at
    src/model/config.cpp:245-249) limits a query to the last `window` keys; it
    exists for the tests of the attention part alone."""
    T, nq, d = q.shape
    group = nq // k.shape[1]
    scale = 1.0 / math.sqrt(d)
    out = np.zeros((T, nq, d), dtype=np.float64)
    for h in range(nq):
        kh, vh = k[:, h // group, :], v[:, h // group, :]
        scores = (q[:, h, :] @ kh.T) * scale
        for p in range(T):
            lo = 0 if window is None else max(0, p - window + 1)
            s = scores[p, lo:p + 1]
            w = np.exp(s - s.max())
            out[p, h, :] = (w @ vh[lo:p + 1]) / w.sum()
    return rnd(out)


def self_attention(x, positions, cfg, w, prefix, cos, sin, rnd=identity):
    """q/k/v projections -> per-head q_norm/k_norm -> RoPE -> attention -> o_proj.
    src/model/self_attention.cpp:122-169"""
    T = x.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = linear(x, w[prefix + "self_attn.q_proj.weight"], rnd).reshape(T, nq, d)
    k = linear(x, w[prefix + "self_attn.k_proj.weight"], rnd).reshape(T, nkv, d)
    v = linear(x, w[prefix + "self_attn.v_proj.weight"], rnd).reshape(T, nkv, d)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps, rnd)     # :147
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps, rnd)     # :149
    q = apply_rope(q, positions, cos, sin, rnd)                           # :152
    k = apply_rope(k, positions, cos, sin, rnd)
    ctx = gqa_attention(q, k, v, rnd).reshape(T, nq * d)                  # :158
    return linear(ctx, w[prefix + "self_attn.o_proj.weight"], rnd)        # :168


def silu_multiply(gate, up, rnd=identity):
    """rnd(rnd(g / (1 + exp(-g))) * u).  src/ops/elementwise.cu:47-65"""
    return rnd(rnd(gate / (1.0 + np.exp(-gate))) * up)


def mlp(x, w, prefix, rnd=identity):
    """down(silu(gate(x)) * up(x)).  src/model/mlp.cpp:101-115"""
    g = linear(x, w[prefix + "mlp.gate_proj.weight"], rnd)
    u = linear(x, w[prefix + "mlp.up_proj.weight"], rnd)
    return linear(silu_multiply(g, u, rnd), w[prefix + "mlp.down_proj.weight"], rnd)


def decoder_layer(x, positions, cfg, w, layer, cos, sin, rnd=identity):
    """x += Attn(RMSNorm(x)); x += MLP(RMSNorm(x)).  src/model/decoder_layer.cpp:63-98"""
    prefix = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    a = rms_norm(x, w[prefix + "input_layernorm.weight"], eps, rnd)                  # :72
    x = rnd(x + self_attention(a, positions, cfg, w, prefix, cos, sin, rnd))        # :78
    m = rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps, rnd)         # :88
    return rnd(x + mlp(m, w, prefix, rnd))                                           # :94


def output_weight(cfg, w):
    """Tied models reuse the embedding table.  src/model/weights.cpp:198-204"""
    return w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]


def forward(cfg, weights, token_ids, rnd=identity, rnd_logits=None, rows=None):
    """Logits [T, V] at every position of one sequence that starts at position 0 (or only at
    the positions `rows`, [len(rows), V]):
    embedding -> layers -> final norm (src/model/model.cpp:107-147) -> output
    projection (src/model/lm_head.cpp:188-191, there for the last row only).
    Every product widens its operands to float64 where it uses them, so large tables may be
    handed over in a narrower type that holds their values exactly."""
    w = weights
    T = len(token_ids)
    positions = np.arange(T)
    cos, sin = rope_table(T, cfg["head_dim"], cfg["rope_theta"])
    x = embedding(token_ids, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, positions, cfg, w, layer, cos, sin, rnd)
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"], rnd)
    return linear(x, output_weight(cfg, w), rnd if rnd_logits is None else rnd_logits)


# ----------------------------------------------------------------------------- sampling


def argmax_lowest(logits, valid=None):
    """Greedy choice: highest logit, lowest id among equals, NaN counts as -inf.
    src/ops/argmax.cu:28-32,58-60"""
    row = np.array(logits[:valid] if valid else logits, dtype=np.float64)
    row[np.isnan(row)] = -np.inf
    return int(np.argmax(row))


def sample_row(logits, temperature, top_k, top_p, u, valid=None):
    """One draw in the reference's order: temperature -> top-k (every candidate
    whose score reaches the k-th best stays) -> sort by score, lower id first among
    equals -> softmax weights exp(score - max) -> shortest prefix whose weight
    reaches top_p of the total -> inverse-CDF draw r = u * kept weight, first
    index with r < cumulative weight.  src/generation/sampler.cpp:137-247"""
    row = np.asarray(logits[:valid] if valid else logits, dtype=np.float64)
    if not np.all(np.isfinite(row)):
        raise RuntimeError("non-finite logit")
    score = row / float(temperature)
    ids = np.arange(row.shape[0])
    if top_k and top_k < row.shape[0]:
        kth = np.sort(score)[::-1][top_k - 1]
        keep = score >= kth
        score, ids = score[keep], ids[keep]
    order = np.lexsort((ids, -score))
    score, ids = score[order], ids[order]
    weights = np.exp(score - score[0])
    total = 0.0
    for x in weights:
        total += x
    threshold = float(top_p) * total
    kept, kept_weight = len(weights), 0.0
    for i, x in enumerate(weights):
        kept_weight += x
        if kept_weight >= threshold:
            kept = i + 1
            break
    r = u * kept_weight
    cumulative = 0.0
    for i in range(kept):
        cumulative += weights[i]
        if r < cumulative:
            return int(ids[i])
    return int(ids[kept - 1])


def generate_greedy(cfg, weights, prompt, max_new_tokens, stop_token_ids=()):
    """The reference's loop for one sequence: logits of the last position ->
    choose -> append -> stop check (the stop token is kept and not fed back).
    src/generation/generator.cpp:272-318"""
    tokens = list(prompt)
    new = []
    for _ in range(max_new_tokens):
        nxt = argmax_lowest(forward(cfg, weights, tokens)[-1])
        new.append(nxt)
        if nxt in stop_token_ids:
            break
        tokens.append(nxt)
    return new
