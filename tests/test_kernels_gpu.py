"""Each kernel alone against its plain formula, at sizes other than the models' (odd widths,
widths that are no multiple of the vector size, head sizes 16..256, several group sizes)."""
import math

import numpy as np
import pytest

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype):
    return torch.as_tensor(np.asarray(a), dtype=torch.float64).to(DT[dtype]).cuda().contiguous()


def back(t):
    return t.detach().to(torch.float64).cpu().numpy()


def stored(a, dtype):
    """The values the device really holds for `a` in `dtype`, as float64."""
    return back(dev(a, dtype))


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == "float32" else 1.2e-2) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,size", [(7, 1000), (3, 1001), (5, 16), (2, 5120), (1, 12)])
def test_rms_norm_with_and_without_residual(dtype, rows, size):
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(rows * size)
    x, d = rng.normal(0, 2, (rows, size)), rng.normal(0, 2, (rows, size))
    w = 1 + rng.normal(0, 0.1, size)
    eps = 3e-5
    rnd = plain.identity if dtype == "float32" else plain.round_bf16
    xs, ds = stored(x, dtype), stored(d, dtype)
    wd = torch.as_tensor(w, dtype=torch.float32).cuda()
    wf = wd.double().cpu().numpy()
    out = torch.empty_like(dev(x, dtype))
    ops.rms_norm(dev(x, dtype), wd, eps, out)
    np.testing.assert_allclose(back(out), plain.rms_norm(xs, wf, eps, rnd), atol=tol(dtype, 4), rtol=tol(dtype))
    xr = dev(x, dtype)
    ops.rms_norm(xr, wd, eps, out, dev(d, dtype))
    summed = rnd(xs + ds)
    np.testing.assert_allclose(back(xr), summed, atol=tol(dtype, 8), rtol=0)
    np.testing.assert_allclose(back(out), plain.rms_norm(summed, wf, eps, rnd), atol=tol(dtype, 4), rtol=tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [64, 100, 7])
def test_embedding_and_gather(dtype, hidden):
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(hidden)
    table = rng.normal(0, 1, (37, hidden))
    ids = rng.integers(0, 37, size=19)
    td = dev(table, dtype)
    out = torch.empty(19, hidden, dtype=DT[dtype], device="cuda")
    ops.embedding(torch.as_tensor(ids, dtype=torch.int32).cuda(), td, out)
    np.testing.assert_array_equal(back(out), plain.embedding(ids, back(td)))
    idx = torch.as_tensor([18, 0, 5, 5], dtype=torch.int32).cuda()
    picked = torch.empty(4, hidden, dtype=DT[dtype], device="cuda")
    ops.gather_rows(out, idx, picked)
    np.testing.assert_array_equal(back(picked), back(out)[[18, 0, 5, 5]])
    delta = dev(rng.normal(0, 1, (19, hidden)), dtype)
    ops.gather_rows(out, idx, picked, delta)
    rnd = plain.identity if dtype == "float32" else plain.round_bf16
    np.testing.assert_allclose(back(picked), rnd((back(out) + back(delta))[[18, 0, 5, 5]]), atol=tol(dtype), rtol=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,inter", [(5, 160), (3, 75), (1, 12288)])
def test_silu_mul(dtype, rows, inter):
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(inter)
    gu = rng.normal(0, 2, (rows, 2 * inter))
    gd = dev(gu, dtype)
    out = torch.empty(rows, inter, dtype=DT[dtype], device="cuda")
    ops.silu_mul(gd, out)
    g = back(gd)
    rnd = plain.identity if dtype == "float32" else plain.round_bf16
    np.testing.assert_allclose(back(out), plain.silu_multiply(g[:, :inter], g[:, inter:], rnd),
                               atol=tol(dtype, 2), rtol=tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 45, 67), (37, 130, 64), (64, 64, 16), (65, 63, 129), (3, 301, 80), (130, 7, 1000)])
def test_gemm_f32_is_true_32_bit(M, N, K):
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(M * N + K)
    x, w = rng.normal(0, 1, (M, K)), rng.normal(0, 1, (N, K))
    xd, wd = dev(x, "float32"), dev(w, "float32")
    out = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.gemm_f32(xd, wd, out)
    exact = back(xd) @ back(wd).T
    # 32-bit accumulation of K products of unit scale: error ~ K * 2^-24 * |terms|; TF32 would be ~1e-3
    assert np.max(np.abs(back(out) - exact)) <= 3e-6 * math.sqrt(K) * 4
    # a row's result does not depend on the other rows of the batch
    one = torch.empty(1, N, dtype=torch.float32, device="cuda")
    ops.gemm_f32(xd[M - 1:M].contiguous(), wd, one)
    assert torch.equal(one[0], out[M - 1])


@pytest.mark.parametrize("M,N,K", [(1, 45, 67), (37, 130, 100), (200, 333, 100), (5, 64, 9)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_bf16_product_of_any_width(M, N, K, out_dtype):
    """Widths that are no multiple of 8 (the tensor-core kernels refuse them): bfloat16 operands, 32-bit sums."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(M * N + K)
    xd, wd = dev(rng.normal(0, 1, (M, K)), "bfloat16"), dev(rng.normal(0, 1, (N, K)), "bfloat16")
    out = torch.full((M, N), float("nan"), dtype=DT[out_dtype], device="cuda")
    ops.gemm_bf16_any_width(xd, wd, out)
    exact = back(xd) @ back(wd).T
    bound = 3e-6 * math.sqrt(K) * 4 if out_dtype == "float32" else 0.02 * math.sqrt(K)
    assert np.max(np.abs(back(out) - exact)) <= bound


def paged_case(rng, lengths, nkv, d, dtype, n_spare=3):
    """Random page tables (shuffled pages) for sequences of the given lengths."""
    pages_per_seq = max(-(-n // 64) for n in lengths)
    n_pages = sum(-(-n // 64) for n in lengths) + n_spare
    order = rng.permutation(n_pages)
    table = np.full((len(lengths), pages_per_seq), -1, dtype=np.int32)
    k = 0
    for s, n in enumerate(lengths):
        for i in range(-(-n // 64)):
            table[s, i] = order[k]
            k += 1
    kp = torch.zeros(n_pages, nkv, 64, d, dtype=DT[dtype], device="cuda")
    vp = torch.zeros_like(kp)
    return table, kp, vp


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 16), (8, 1, 32), (6, 3, 48), (8, 2, 128), (2, 2, 256), (5, 5, 80)])
def test_prepare_and_attention_over_pages(dtype, nq, nkv, d):
    """Two steps per sequence (a prompt, then more tokens) through qkv_prepare and the attention
    kernel, over shuffled pages, against per-head norm + rotation + causal attention in float64."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(nq * 1000 + d)
    lengths, first = [70, 5, 129], [64, 1, 100]
    eps, theta = 2e-5, 12345.0
    rnd = plain.identity if dtype == "float32" else plain.round_bf16
    table, kp, vp = paged_case(rng, lengths, nkv, d, dtype)
    table_d = torch.as_tensor(table).cuda()
    cos, sin = plain.rope_table(max(lengths), d, theta)
    cos_d = torch.as_tensor(cos, dtype=torch.float32).cuda()
    sin_d = torch.as_tensor(sin, dtype=torch.float32).cuda()
    qw, kw = 1 + rng.normal(0, 0.1, d), 1 + rng.normal(0, 0.1, d)
    qw_d, kw_d = torch.as_tensor(qw, dtype=torch.float32).cuda(), torch.as_tensor(kw, dtype=torch.float32).cuda()
    qw, kw = qw_d.double().cpu().numpy(), kw_d.double().cpu().numpy()
    full = [rng.normal(0, 1, (n, (nq + 2 * nkv) * d)) for n in lengths]
    got = [np.zeros((n, nq * d)) for n in lengths]
    for part in range(2):
        spans = [(0, f) if part == 0 else (f, n) for f, n in zip(first, lengths)]
        rows = np.concatenate([full[s][a:b] for s, (a, b) in enumerate(spans)])
        seq = np.concatenate([np.full(b - a, s) for s, (a, b) in enumerate(spans)]).astype(np.int32)
        pos = np.concatenate([np.arange(a, b) for a, b in spans]).astype(np.int32)
        N = rows.shape[0]
        qkv = dev(rows, dtype)
        q = torch.empty(N, nq * d, dtype=DT[dtype], device="cuda")
        out = torch.empty_like(q)
        seq_d, pos_d = torch.as_tensor(seq).cuda(), torch.as_tensor(pos).cuda()
        ops.qkv_prepare(qkv, q, kp, vp, qw_d, kw_d, cos_d, sin_d, seq_d, pos_d, table_d, N, nq, nkv, d, eps)
        ops.attention_generic(q, kp, vp, out, seq_d, pos_d, table_d, N, nq, nkv, d, d ** -0.5)
        o = back(out)
        k = 0
        for s, (a, b) in enumerate(spans):
            got[s][a:b] = o[k:k + b - a]
            k += b - a
    for s, n in enumerate(lengths):
        x = stored(full[s], dtype)
        qs = x[:, :nq * d].reshape(n, nq, d)
        ks = x[:, nq * d:(nq + nkv) * d].reshape(n, nkv, d)
        vs = x[:, (nq + nkv) * d:].reshape(n, nkv, d)
        pos = np.arange(n)
        qs = plain.apply_rope(plain.rms_norm(qs, qw, eps, rnd), pos, cos, sin, rnd)
        ks = plain.apply_rope(plain.rms_norm(ks, kw, eps, rnd), pos, cos, sin, rnd)
        want = plain.gqa_attention(qs, ks, vs).reshape(n, nq * d)
        err = np.max(np.abs(got[s] - want))
        assert err <= tol(dtype, 3), f"sequence {s}: max abs err {err:.3e}"
        # the cache holds the rotated keys and the raw values at the right page and row
        for p in (0, n - 1, min(n - 1, 64)):
            page = table[s, p // 64]
            np.testing.assert_allclose(back(kp[page, :, p % 64, :]), ks[p], atol=tol(dtype, 3), rtol=0)
            np.testing.assert_array_equal(back(vp[page, :, p % 64, :]), vs[p])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """One early key is made to dominate one late query: the output must be that key's value.
    Random keys alone would hide a kernel that skips a page or reads a wrong row."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(5)
    nq, nkv, d, n = 4, 2, 32, 600
    for far in (3, 64, 127, 320, 598):
        table, kp, vp = paged_case(rng, [n], nkv, d, dtype)
        rows = rng.normal(0, 0.3, (n, (nq + 2 * nkv) * d))
        direction = rng.normal(0, 1, d)
        direction *= 12.0 / np.linalg.norm(direction)
        rows[n - 1, 2 * d:3 * d] = direction * 3             # query head 2 (kv head 1) of the last token
        rows[far, (nq + 1) * d:(nq + 2) * d] = direction * 3    # key of kv head 1 at `far`
        seq = torch.zeros(n, dtype=torch.int32, device="cuda")
        pos = torch.arange(n, dtype=torch.int32, device="cuda")
        q = torch.empty(n, nq * d, dtype=DT[dtype], device="cuda")
        out = torch.empty_like(q)
        table_d = torch.as_tensor(table).cuda()
        ops.qkv_prepare(dev(rows, dtype), q, kp, vp, None, None, None, None, seq, pos, table_d, n, nq, nkv, d, 0.0)
        ops.attention_generic(q, kp, vp, out, seq, pos, table_d, n, nq, nkv, d, d ** -0.5)
        x = stored(rows, dtype)
        value = x[far, (nq + nkv + 1) * d:(nq + nkv + 2) * d]
        got = back(out)[n - 1, 2 * d:3 * d]
        assert np.max(np.abs(got - value)) <= 2e-2, f"far key {far}: {np.max(np.abs(got - value)):.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_window_edge(dtype):
    """With a window of w keys, a dominating key exactly w back is invisible and one w-1 back is seen."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(6)
    nq, nkv, d, n, window = 2, 1, 16, 200, 70
    for back_by, seen in ((window - 1, True), (window, False)):
        table, kp, vp = paged_case(rng, [n], nkv, d, dtype)
        rows = rng.normal(0, 0.3, (n, (nq + 2 * nkv) * d))
        direction = rng.normal(0, 1, d)
        direction *= 36.0 / np.linalg.norm(direction)
        far = n - 1 - back_by
        rows[n - 1, 0:d] = direction
        rows[far, nq * d:(nq + 1) * d] = direction
        seq = torch.zeros(n, dtype=torch.int32, device="cuda")
        pos = torch.arange(n, dtype=torch.int32, device="cuda")
        q = torch.empty(n, nq * d, dtype=DT[dtype], device="cuda")
        out = torch.empty_like(q)
        table_d = torch.as_tensor(table).cuda()
        ops.qkv_prepare(dev(rows, dtype), q, kp, vp, None, None, None, None, seq, pos, table_d, n, nq, nkv, d, 0.0)
        ops.attention_generic(q, kp, vp, out, seq, pos, table_d, n, nq, nkv, d, d ** -0.5, window)
        x = stored(rows, dtype)
        qs = x[:, :nq * d].reshape(n, nq, d)
        ks = x[:, nq * d:(nq + nkv) * d].reshape(n, nkv, d)
        vs = x[:, (nq + nkv) * d:].reshape(n, nkv, d)
        want = plain.gqa_attention(qs, ks, vs, window=window).reshape(n, nq * d)
        assert np.max(np.abs(back(out) - want)) <= tol(dtype, 3)
        hit = np.max(np.abs(back(out)[n - 1, :d] - vs[far, 0])) <= 2e-2
        assert hit == seen


def test_argmax_lowest_id_among_equals_and_nan():
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(7)
    logits = rng.normal(0, 1, (6, 1013)).astype(np.float32)
    logits[0, [400, 17, 900]] = 9.0
    logits[1, 5] = np.nan
    logits[2, :] = -np.inf
    logits[3, 1012] = 50.0
    logits[4, 0] = 50.0
    logits[5, 700:] = 100.0            # beyond the valid prefix in the second call
    d = torch.as_tensor(logits).cuda()
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.argmax(d, out)
    assert out.tolist() == [plain.argmax_lowest(r) for r in logits]
    assert out.tolist()[:5] == [17, plain.argmax_lowest(logits[1]), 0, 1012, 0]
    ops.argmax(d, out, 700)
    assert out.tolist() == [plain.argmax_lowest(r, 700) for r in logits]


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.6, 20, 0.95), (1.0, 0, 1.0), (0.7, 0, 0.9), (1.3, 5, 1.0),
                                                     (0.2, 1, 0.5), (2.0, 300, 0.3), (0.9, 1200, 0.8)])
@pytest.mark.parametrize("vocab,valid", [(1500, 1400), (20011, 20000)])
def test_sampling_kernel_follows_the_reference_order(temperature, top_k, top_p, vocab, valid):
    """The kernel's draw equals the plain walk (temperature -> top-k with ties -> sort -> softmax
    -> top-p -> inverse CDF) for the same uniform number, on rows with many equal logits."""
    from qwen3_b200 import uniform_for
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(int(temperature * 10) + top_k)
    rows = 24 if vocab < 10000 else 8
    logits = rng.normal(0, 2.5, (rows, vocab)).astype(np.float32)
    logits[::2] = np.round(logits[::2] * 4) / 4          # coarse values: many ties, as bfloat16 logits have
    logits[:, valid:] = 1e4                              # ids beyond the valid prefix must never be drawn
    logits[3, :50] = 6.0
    seed = 42
    seq_ids = torch.arange(100, 100 + rows, dtype=torch.int64, device="cuda")
    d = torch.as_tensor(logits).cuda()
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    for step in (0, 1, 7):
        steps = torch.full((rows,), step, dtype=torch.int32, device="cuda")
        ops.sample(d, out, temperature, top_k, top_p, seed, seq_ids, steps, valid)
        got = out.tolist()
        want = [plain.sample_row(logits[r], np.float32(temperature), top_k, np.float32(top_p),
                                 uniform_for(seed, 100 + r, step), valid) for r in range(rows)]
        assert got == want, (step, got, want)
    ops.sample(d, out, temperature, top_k, top_p, seed, seq_ids, 7, valid)       # one step number for all rows
    assert out.tolist() == want
    # a row's draw does not depend on how many rows share the launch (the blocks per row do)
    for part in (3, min(rows, 20)):
        ops.sample(d[:part], out[:part], temperature, top_k, top_p, seed, seq_ids[:part], 7, valid)
        assert out[:part].tolist() == want[:part]
    many = d.repeat(10, 1)
    out_many = torch.empty(many.shape[0], dtype=torch.int32, device="cuda")
    ops.sample(many, out_many, temperature, top_k, top_p, seed, seq_ids.repeat(10), 7, valid)
    assert out_many.tolist() == want * 10
    bad = logits.copy()
    bad[2, 7] = np.inf
    ops.sample(torch.as_tensor(bad).cuda(), out, temperature, top_k, top_p, seed, seq_ids, steps, valid)
    assert out.tolist()[2] == -1 and out.tolist()[1] == want[1]


def test_sampling_statistics_match_the_distribution():
    """Over many streams the kernel's draws follow softmax(logits / T) restricted by top-k."""
    from qwen3_b200.csrc import ops
    logits = np.array([[2.0, 2.0, 1.0, -10.0, 0.5, 0.0, -1.0, 1.5]], dtype=np.float32)
    n = 4000
    d = torch.as_tensor(np.repeat(logits, n, axis=0)).cuda()
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(d, out, 0.8, 3, 1.0, 9, torch.arange(n, dtype=torch.int64, device="cuda"),
               torch.zeros(n, dtype=torch.int32, device="cuda"))
    counts = np.bincount(out.cpu().numpy(), minlength=8)
    assert counts[[2, 3, 4, 5, 6]].sum() == 0            # top-3 keeps ids 0, 1 (tie) and 7
    w = np.exp(np.array([2.0, 2.0, 1.5]) / 0.8)
    expect = w / w.sum() * n
    assert np.all(np.abs(counts[[0, 1, 7]] - expect) < 5 * np.sqrt(expect))


@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (3, 301, 80), (8, 130, 1024), (9, 96, 288), (16, 4100, 512),
                                   (17, 50, 4096), (33, 77, 160), (64, 1030, 2048), (5, 9600, 96), (12, 20000, 64)])
def test_skinny_product(M, N, K, out_dtype):
    """The weight-streaming kernel against float64, for every batch-row tile count, row-tile
    count and K tail, and with rows that do not depend on the rest of the batch."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(M + N + K)
    xd, wd = dev(rng.normal(0, 1, (M, K)), "bfloat16"), dev(rng.normal(0, 1, (N, K)), "bfloat16")
    out = torch.empty(M, N, dtype=DT[out_dtype], device="cuda")
    ops.gemm_skinny(xd, wd, out)
    exact = back(xd) @ back(wd).T
    if out_dtype == "float32":
        assert np.max(np.abs(back(out) - exact)) <= 2e-5 * math.sqrt(K) * 4
    else:
        np.testing.assert_allclose(back(out), exact, atol=1e-2 * math.sqrt(K) / 8, rtol=8e-3)
    one = torch.empty(1, N, dtype=DT[out_dtype], device="cuda")
    ops.gemm_skinny(xd[M - 1:M].contiguous(), wd, one)
    assert torch.equal(one[0], out[M - 1])


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 16), (8, 1, 32), (6, 3, 48), (32, 8, 128), (16, 1, 64), (2, 2, 256), (5, 5, 80)])
def test_decode_attention_split_kernel(nq, nkv, d):
    """One new token per sequence against caches of very different lengths, for several split
    counts, over shuffled pages: equal to float64 attention over the stored bfloat16 values."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(nq + d)
    lengths = [1, 63, 64, 65, 130, 700, 1000]
    table, kp, vp = paged_case(rng, lengths, nkv, d, "bfloat16")
    table_d = torch.as_tensor(table).cuda()
    keys = [rng.normal(0, 1, (n, nkv, d)) for n in lengths]
    vals = [rng.normal(0, 1, (n, nkv, d)) for n in lengths]
    for s, n in enumerate(lengths):
        pages = table[s, :-(-n // 64)]
        kpad = np.zeros((len(pages) * 64, nkv, d)); kpad[:n] = keys[s]
        vpad = np.zeros((len(pages) * 64, nkv, d)); vpad[:n] = vals[s]
        kp[torch.as_tensor(pages).long().cuda()] = dev(kpad.reshape(len(pages), 64, nkv, d).transpose(0, 2, 1, 3), "bfloat16")
        vp[torch.as_tensor(pages).long().cuda()] = dev(vpad.reshape(len(pages), 64, nkv, d).transpose(0, 2, 1, 3), "bfloat16")
    B = len(lengths)
    q = rng.normal(0, 1, (B, nq, d))
    q[5] *= 3.0
    qd = dev(q.reshape(B, nq * d), "bfloat16")
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    pos = torch.as_tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    want = np.zeros((B, nq * d))
    for s, n in enumerate(lengths):
        qs = np.zeros((n, nq, d))
        qs[n - 1] = back(qd)[s].reshape(nq, d)
        want[s] = plain.gqa_attention(qs, stored(keys[s], "bfloat16"), stored(vals[s], "bfloat16"))[n - 1].reshape(-1)
    for splits in (1, 2, 5, 32):
        out = torch.zeros(B, nq * d, dtype=torch.bfloat16, device="cuda")
        scratch = torch.full((B * nq * splits * (d + 2),), float("nan"), dtype=torch.float32, device="cuda")
        ops.attention_decode(qd, kp, vp, out, scratch, seq, pos, table_d, B, nq, nkv, d, d ** -0.5, None, splits)
        err = np.max(np.abs(back(out) - want))
        assert err <= 1.5e-2, f"splits {splits}: max abs err {err:.3e}"
    # the generic kernel agrees on the same cache
    out2 = torch.zeros_like(out)
    ops.attention_generic(qd, kp, vp, out2, seq, pos, table_d, B, nq, nkv, d, d ** -0.5)
    assert np.max(np.abs(back(out2) - want)) <= 1.5e-2
    # a window of 100 keys
    out3 = torch.zeros_like(out)
    scratch = torch.zeros(B * nq * 3 * (d + 2), dtype=torch.float32, device="cuda")
    ops.attention_decode(qd, kp, vp, out3, scratch, seq, pos, table_d, B, nq, nkv, d, d ** -0.5, 100, 3)
    ops.attention_generic(qd, kp, vp, out2, seq, pos, table_d, B, nq, nkv, d, d ** -0.5, 100)
    assert np.max(np.abs(back(out3) - back(out2))) <= 1.5e-2
    assert np.max(np.abs(back(out3)[6] - want[6])) > 1e-3      # the window really hides the older keys


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 16), (8, 1, 32), (6, 3, 48), (32, 8, 128), (16, 1, 64), (2, 2, 256), (5, 5, 80)])
def test_decode_attention_fused_kernel(nq, nkv, d):
    """The whole attention of a decode step in one launch, from the raw projection output: equal to the plain
    per-head norm, rotation and attention in float64 with the reference's rounding points, for several split
    counts; the new key and value land in the cache, at the right place of the right page and nowhere else;
    a far key is scaled so that it stands out among hundreds, and the query norm doubles half of every head."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(3 * nq + d)
    lengths = [1, 63, 64, 65, 130, 700, 1000]
    eps, theta = 1e-5, 50000.0
    table, kp, vp = paged_case(rng, lengths, nkv, d, "bfloat16")
    table_d = torch.as_tensor(table).cuda()
    keys = [rng.normal(0, 1, (n, nkv, d)) for n in lengths]       # the last row of each is overwritten by the step
    vals = [rng.normal(0, 1, (n, nkv, d)) for n in lengths]
    keys[5][17] *= 4.0                                            # a far key of sequence 5 ...
    for s, n in enumerate(lengths):
        pages = table[s, :-(-n // 64)]
        kpad = np.zeros((len(pages) * 64, nkv, d)); kpad[:n - 1] = keys[s][:n - 1]
        vpad = np.zeros((len(pages) * 64, nkv, d)); vpad[:n - 1] = vals[s][:n - 1]
        kp[torch.as_tensor(pages).long().cuda()] = dev(kpad.reshape(len(pages), 64, nkv, d).transpose(0, 2, 1, 3), "bfloat16")
        vp[torch.as_tensor(pages).long().cuda()] = dev(vpad.reshape(len(pages), 64, nkv, d).transpose(0, 2, 1, 3), "bfloat16")
    B = len(lengths)
    qkv = rng.normal(0, 1, (B, (nq + 2 * nkv) * d))
    qkv_d = dev(qkv, "bfloat16")
    qw, kw = 1.0 + 0.1 * rng.normal(size=d), 1.0 + 0.1 * rng.normal(size=d)
    qw[: d // 2] *= 2.0                                           # ... and a query norm that doubles half of every head
    cos, sin = plain.rope_table(max(lengths), d, theta)
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    pos = torch.as_tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    rnd = plain.round_bf16
    raw = back(qkv_d)
    want = np.zeros((B, nq * d))
    new_k, new_v = [], []
    for s, n in enumerate(lengths):
        q = plain.rms_norm(raw[s, :nq * d].reshape(1, nq, d), qw.astype(np.float32).astype(np.float64), eps, rnd)
        k = plain.rms_norm(raw[s, nq * d:(nq + nkv) * d].reshape(1, nkv, d), kw.astype(np.float32).astype(np.float64), eps, rnd)
        q = plain.apply_rope(q, np.array([n - 1]), cos, sin, rnd)
        k = plain.apply_rope(k, np.array([n - 1]), cos, sin, rnd)
        v = raw[s, (nq + nkv) * d:].reshape(1, nkv, d)
        new_k.append(k[0]); new_v.append(v[0])
        ks, vs = stored(keys[s], "bfloat16"), stored(vals[s], "bfloat16")
        ks[n - 1], vs[n - 1] = k[0], v[0]
        qs = np.zeros((n, nq, d)); qs[n - 1] = q[0]
        want[s] = plain.gqa_attention(qs, ks, vs)[n - 1].reshape(-1)
    before_k, before_v = kp.clone(), vp.clone()
    args = (dev(qw, "float32"), dev(kw, "float32"), dev(cos, "float32"), dev(sin, "float32"), eps, seq, pos, table_d, B, nq, nkv, d,
            d ** -0.5, None)
    for splits in (1, 2, 5, 8, 11, 16):
        kp.copy_(before_k); vp.copy_(before_v)
        out = torch.zeros(B, nq * d, dtype=torch.bfloat16, device="cuda")
        ops.attention_decode_fused(qkv_d, kp, vp, out, *args, splits)
        err = np.max(np.abs(back(out) - want))
        assert err <= 2.5e-2, f"splits {splits}: max abs err {err:.3e}"      # the tolerance of the decode kernel, plus the rounding of q
    # the cache: only the new token's row of every (sequence, kv head) changed, to the plain values
    changed_k, changed_v = (kp != before_k).any(dim=-1), (vp != before_v).any(dim=-1)      # [page, kv head, slot]
    expect = torch.zeros_like(changed_k)
    for s, n in enumerate(lengths):
        page, slot = int(table[s, (n - 1) // 64]), (n - 1) % 64
        expect[page, :, slot] = True
        assert np.max(np.abs(back(kp[page, :, slot]) - new_k[s])) <= 1e-6 + 2.0 ** -7 * np.max(np.abs(new_k[s])), s
        assert np.array_equal(back(vp[page, :, slot]), new_v[s]), s
    assert torch.equal(changed_k | changed_v, expect)
    # a layer that reads another layer's cache writes nothing and finds the new key and value there
    out2 = torch.zeros_like(out)
    snapshot_k, snapshot_v = kp.clone(), vp.clone()
    ops.attention_decode_fused(qkv_d, kp, vp, out2, *args, 3, write_kv=False)
    assert torch.equal(kp, snapshot_k) and torch.equal(vp, snapshot_v)
    assert np.max(np.abs(back(out2) - want)) <= 2.5e-2
    with pytest.raises(ops.KernelError):
        ops.attention_decode_fused(qkv_d, kp, vp, out2, *args, 17)


@pytest.mark.parametrize("nq,nkv,d,rot", [(4, 2, 64, 32), (8, 1, 128, 64), (6, 3, 48, 16), (5, 5, 80, 2), (2, 2, 256, 254),
                                          (3, 1, 96, 96)])
def test_partial_rotation_stays_fused(nq, nkv, d, rot):
    """Tables of width rot/2 rotate only the first `rot` values of a head, in pairs (i, i + rot/2); the rest is
    normalised and passes through.  The prepare kernel in 32-bit and in bfloat16 (a prompt of more and of fewer
    than 64 tokens) and the one-launch decode attention agree with the plain float64 norm and rotation; the decode
    step's new key is the one the prepare kernel would have written, to the bit.  The inputs make a fault show: the
    values from `rot` on are ten times larger than the rotated ones, so rotating or dropping one of them is far
    outside the tolerance."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(d + rot)
    eps, theta = 3e-6, 777.0
    lengths = [150, 9]
    cos, sin = plain.rope_table(max(lengths) + 1, rot, theta)
    assert cos.shape[1] == rot // 2
    cos_d, sin_d = dev(cos, "float32"), dev(sin, "float32")
    qw, kw = 1 + rng.normal(0, 0.1, d), 1 + rng.normal(0, 0.1, d)
    qw_d, kw_d = dev(qw, "float32"), dev(kw, "float32")
    qw, kw = qw_d.double().cpu().numpy(), kw_d.double().cpu().numpy()
    full = [rng.normal(0, 1, (n + 1, nq + 2 * nkv, d)) for n in lengths]      # the last row is the decode step's
    for x in full:
        x[..., rot:] *= 10.0
    full = [x.reshape(x.shape[0], -1) for x in full]
    seq = np.concatenate([np.full(n, s) for s, n in enumerate(lengths)]).astype(np.int32)
    pos = np.concatenate([np.arange(n) for n in lengths]).astype(np.int32)
    N = len(seq)
    seq_d, pos_d = torch.as_tensor(seq).cuda(), torch.as_tensor(pos).cuda()
    for dtype in ("float32", "bfloat16"):
        rnd = plain.identity if dtype == "float32" else plain.round_bf16
        table, kp, vp = paged_case(rng, [n + 1 for n in lengths], nkv, d, dtype)
        table_d = torch.as_tensor(table).cuda()
        qkv = dev(np.concatenate([x[:-1] for x in full]), dtype)
        q = torch.empty(N, nq * d, dtype=DT[dtype], device="cuda")
        ops.qkv_prepare(qkv, q, kp, vp, qw_d, kw_d, cos_d, sin_d, seq_d, pos_d, table_d, N, nq, nkv, d, eps)
        got_q = back(q)
        row = 0
        wants = []
        for s, n in enumerate(lengths):
            x = stored(full[s], dtype)
            qs = x[:, :nq * d].reshape(n + 1, nq, d)
            ks = x[:, nq * d:(nq + nkv) * d].reshape(n + 1, nkv, d)
            vs = x[:, (nq + nkv) * d:].reshape(n + 1, nkv, d)
            p = np.arange(n + 1)
            qs = plain.apply_rope(plain.rms_norm(qs, qw, eps, rnd), p, cos, sin, rnd)
            ks = plain.apply_rope(plain.rms_norm(ks, kw, eps, rnd), p, cos, sin, rnd)
            wants.append((qs, ks, vs))
            scale = np.max(np.abs(qs))
            assert np.max(np.abs(got_q[row:row + n] - qs[:n].reshape(n, -1))) <= tol(dtype, 3) * scale, (dtype, s)
            for t in (0, n - 1, min(n - 1, 64)):
                page = table[s, t // 64]
                assert np.max(np.abs(back(kp[page, :, t % 64]) - ks[t])) <= tol(dtype, 3) * scale, (dtype, s, t)
                np.testing.assert_array_equal(back(vp[page, :, t % 64]), vs[t])
            row += n
    # the decode step of both sequences in one launch (bfloat16; kp, vp and wants are the bfloat16 ones)
    B = len(lengths)
    step = dev(np.stack([x[-1] for x in full]), "bfloat16")
    dseq = torch.arange(B, dtype=torch.int32, device="cuda")
    dpos = torch.as_tensor(lengths, dtype=torch.int32).cuda()
    out = torch.zeros(B, nq * d, dtype=torch.bfloat16, device="cuda")
    kp2, vp2 = kp.clone(), vp.clone()
    ops.attention_decode_fused(step, kp, vp, out, qw_d, kw_d, cos_d, sin_d, eps, dseq, dpos, table_d, B, nq, nkv, d, d ** -0.5,
                               None, 2)
    q2 = torch.empty(B, nq * d, dtype=torch.bfloat16, device="cuda")
    ops.qkv_prepare(step, q2, kp2, vp2, qw_d, kw_d, cos_d, sin_d, dseq, dpos, table_d, B, nq, nkv, d, eps)
    assert torch.equal(kp, kp2) and torch.equal(vp, vp2)
    for s, n in enumerate(lengths):
        qs, ks, vs = wants[s]
        want = plain.gqa_attention(qs, ks, vs)[n].reshape(-1)
        assert np.max(np.abs(back(out[s]) - want)) <= 2.5e-2 * max(1.0, np.max(np.abs(vs))), s
    # tables that are wider than the head are refused
    wide = torch.zeros(8, d // 2 + 1, dtype=torch.float32, device="cuda")
    with pytest.raises(ops.KernelError):
        ops.qkv_prepare(step, q2, kp2, vp2, qw_d, kw_d, wide, wide, dseq, dpos, table_d, B, nq, nkv, d, eps)


@pytest.mark.parametrize("nq,nkv,d", [(4, 2, 16), (8, 1, 32), (6, 3, 48), (8, 2, 128), (2, 2, 256), (5, 5, 80)])
@pytest.mark.parametrize("window", [None, 90])
def test_prefill_attention_tiled_kernel(nq, nkv, d, window):
    """Prompts of unequal length in one launch, then a second launch that continues them from the
    cache (positions > 0, tiles that straddle page edges), against float64 causal attention."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(nq * 31 + d)
    lengths, first = [200, 5, 129, 64, 333], [64, 1, 100, 63, 130]
    table, kp, vp = paged_case(rng, lengths, nkv, d, "bfloat16")
    table_d = torch.as_tensor(table).cuda()
    full = [rng.normal(0, 1, (n, (nq + 2 * nkv) * d)) for n in lengths]
    got = [np.zeros((n, nq * d)) for n in lengths]
    for part in range(2):
        spans = [(0, f) if part == 0 else (f, n) for f, n in zip(first, lengths)]
        rows = np.concatenate([full[s][a:b] for s, (a, b) in enumerate(spans)])
        seq = np.concatenate([np.full(b - a, s) for s, (a, b) in enumerate(spans)]).astype(np.int32)
        pos = np.concatenate([np.arange(a, b) for a, b in spans]).astype(np.int32)
        starts = np.cumsum([0] + [b - a for a, b in spans]).astype(np.int32)
        N = rows.shape[0]
        q = torch.empty(N, nq * d, dtype=torch.bfloat16, device="cuda")
        out = torch.zeros_like(q)
        seq_d, pos_d = torch.as_tensor(seq).cuda(), torch.as_tensor(pos).cuda()
        ops.qkv_prepare(dev(rows, "bfloat16"), q, kp, vp, None, None, None, None, seq_d, pos_d, table_d, N, nq, nkv, d, 0.0)
        ops.attention_prefill(q, kp, vp, out, torch.as_tensor(starts).cuda(),
                              torch.as_tensor([a for a, _ in spans], dtype=torch.int32).cuda(), table_d, len(lengths),
                              max(b - a for a, b in spans), nq, nkv, d, d ** -0.5, window)
        o = back(out)
        k = 0
        for s, (a, b) in enumerate(spans):
            got[s][a:b] = o[k:k + b - a]
            k += b - a
    for s, n in enumerate(lengths):
        x = stored(full[s], "bfloat16")
        qs = x[:, :nq * d].reshape(n, nq, d)
        ks = x[:, nq * d:(nq + nkv) * d].reshape(n, nkv, d)
        vs = x[:, (nq + nkv) * d:].reshape(n, nkv, d)
        want = plain.gqa_attention(qs, ks, vs, window=window).reshape(n, nq * d)
        err = np.abs(got[s] - want).max(axis=1)
        assert err.max() <= 2e-2, f"sequence {s}: row {int(err.argmax())} of {n}: max abs err {err.max():.3e}"


@pytest.mark.parametrize("M,N,K", [(16, 128, 64), (1, 128, 64), (5, 256, 128), (17, 200, 80), (64, 384, 512),
                                   (100, 301, 96), (128, 128, 4096), (33, 1000, 1000), (64, 4096, 4096), (24, 130, 12288),
                                   (129, 200, 136), (256, 512, 2048), (300, 1000, 1024), (700, 130, 520)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_tcgen05_weights_first_product(M, N, K, out_dtype):
    """The weights-first TMA + tcgen05 kernel against a 32-bit product of the same bfloat16 operands: every
    token tile, ragged edges in all three dimensions, K that is no multiple of 64, and K split over clusters
    of every size that fits (1 = no cluster reduction, 3 = uneven ranges, 8 = the largest)."""
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    want = (x.double() @ w.double().T)
    for splits in (0, 1, 2, 3, 8):
        out = torch.full((M, N), float("nan"), dtype=DT[out_dtype], device="cuda")
        ops.gemm_tcgen05_mid(x, w, out, splits=splits)
        assert ops.tcgen05_status("cuda") == 0, f"a wait inside the kernel gave up ({splits} K ranges)"
        err = (out.double() - want).abs().max().item()
        bound = 4e-5 * math.sqrt(K) * 4 if out_dtype == "float32" else 0.02 * math.sqrt(K)
        assert err <= bound, f"{splits} K ranges: max abs err {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("M,inter,K", [(17, 64, 64), (64, 12288, 512), (33, 160, 96), (128, 1000, 256), (40, 112, 1000),
                                       (200, 160, 1024), (513, 72, 96)])
def test_tcgen05_weights_first_gated(M, inter, K):
    """The same kernel with SiLU and gating where the partial tiles are added equals product + silu_mul,
    bit for bit at the same number of K ranges, and the plain formula within bfloat16 rounding."""
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(M + inter + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    gate = (torch.randn(inter, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    up = (torch.randn(inter, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate, up)
    gd = plain.round_bf16(back(x) @ back(gate).T)
    ud = plain.round_bf16(back(x) @ back(up).T)
    want = plain.silu_multiply(gd, ud, plain.round_bf16)
    scale = max(1.0, float(np.abs(want).max()))
    for splits in (0, 1, 4):
        fused = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.gemm_tcgen05_mid_gated(x, w, fused, splits=splits)
        gate_up = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device="cuda")
        ops.gemm_tcgen05_mid(x, w, gate_up, splits=splits)
        two = torch.empty_like(fused)
        ops.silu_mul(gate_up, two, interleaved=True)
        assert ops.tcgen05_status("cuda") == 0
        assert torch.equal(fused, two)
        assert np.max(np.abs(back(fused) - want)) <= 2e-2 * scale


@pytest.mark.parametrize("M,inter,K", [(1, 64, 64), (8, 12288, 4096), (3, 160, 96), (16, 1000, 256), (9, 112, 80)])
def test_gated_skinny_product_and_interleaved_silu(M, inter, K):
    """gate/up rows interleaved in blocks of eight: the fused kernel (product + SiLU + gating) and the
    two-kernel path (product, then silu_mul on the interleaved layout) agree with the plain formula."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(M + inter + K)
    xd = dev(rng.normal(0, 1, (M, K)), "bfloat16")
    gate, up = dev(rng.normal(0, 0.2, (inter, K)), "bfloat16"), dev(rng.normal(0, 0.2, (inter, K)), "bfloat16")
    w = ops.interleave_gate_up(gate, up)
    g = plain.round_bf16(back(xd) @ back(gate).T)
    u = plain.round_bf16(back(xd) @ back(up).T)
    want = plain.silu_multiply(g, u, plain.round_bf16)
    fused = torch.empty(M, inter, dtype=torch.bfloat16, device="cuda")
    ops.gemm_skinny_gated(xd, w, fused)
    gate_up = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device="cuda")
    ops.gemm_skinny(xd, w, gate_up)
    two = torch.empty_like(fused)
    ops.silu_mul(gate_up, two, interleaved=True)
    scale = max(1.0, float(np.abs(want).max()))
    assert np.max(np.abs(back(fused) - want)) <= 2e-2 * scale
    assert np.max(np.abs(back(two) - want)) <= 2e-2 * scale
    assert torch.equal(fused, two)                      # same sums, same rounding points
    # and the 32-bit elementwise kernel on the interleaved layout
    gu32 = torch.tensor(rng.normal(0, 2, (M, 2 * inter)), dtype=torch.float32, device="cuda")
    out32 = torch.empty(M, inter, dtype=torch.float32, device="cuda")
    ops.silu_mul(gu32, out32, interleaved=True)
    blocks = back(gu32).reshape(M, inter // 8, 2, 8)
    np.testing.assert_allclose(back(out32), plain.silu_multiply(blocks[:, :, 0, :].reshape(M, inter),
                                                                blocks[:, :, 1, :].reshape(M, inter)), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 8, 64), (200, 301, 80), (2048, 1024, 512), (1000, 6144, 4096),
                                   (4100, 520, 136), (129, 257, 8)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_tcgen05_prompt_product(M, N, K, out_dtype):
    """The persistent tokens-first kernel: many tiles per block (both accumulators in use, the
    stage ring wrapping across tiles), ragged edges, widths that rule out vector stores."""
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(M + 3 * N + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    want = x.double() @ w.double().T
    for tile in (128, 256):
        out = torch.full((M, N), float("nan"), dtype=DT[out_dtype], device="cuda")
        ops.gemm_tcgen05_prompt(x, w, out, tile_n=tile)
        assert ops.tcgen05_status("cuda") == 0, f"a wait inside the kernel gave up (tile {tile})"
        err = (out.double() - want).abs().max().item()
        bound = 4e-5 * math.sqrt(K) * 4 if out_dtype == "float32" else 0.02 * math.sqrt(K)
        assert err <= bound, f"tile {tile}: max abs err {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1, 8, 64), (200, 301, 80), (2048, 1024, 512), (1000, 6144, 4096),
                                   (4100, 520, 136), (129, 257, 8), (300, 40000, 128)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_tcgen05_pair_product(M, N, K, out_dtype):
    """The product on pairs of SMs (cta_group::2): one tile and many per pair, ragged edges (a second block
    whose tokens are all beyond M included), widths that rule out vector stores."""
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(M + 3 * N + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.full((M, N), float("nan"), dtype=DT[out_dtype], device="cuda")
    ops.gemm_tcgen05_pair(x, w, out)
    assert ops.tcgen05_status("cuda") == 0, "a wait inside the kernel gave up"
    err = (out.double() - want).abs().max().item()
    bound = 4e-5 * math.sqrt(K) * 4 if out_dtype == "float32" else 0.02 * math.sqrt(K)
    assert err <= bound, f"max abs err {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("M,inter,K", [(128, 128, 64), (300, 160, 96), (2048, 1536, 512), (77, 112, 80)])
def test_tcgen05_pair_gated_epilogue(M, inter, K):
    """The pair kernel with SiLU and gating in its epilogue equals its own product + silu_mul, bit for bit."""
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(M + inter + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    gate = (torch.randn(inter, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    up = (torch.randn(inter, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate, up)
    fused = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05_pair(x, w, fused, gated=True)
    gate_up = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05_pair(x, w, gate_up)
    two = torch.empty_like(fused)
    ops.silu_mul(gate_up, two, interleaved=True)
    assert ops.tcgen05_status("cuda") == 0
    assert torch.equal(fused, two)
    gd = plain.round_bf16(back(x) @ back(gate).T)
    ud = plain.round_bf16(back(x) @ back(up).T)
    want = plain.silu_multiply(gd, ud, plain.round_bf16)
    assert np.max(np.abs(back(fused) - want)) <= 2e-2 * max(1.0, float(np.abs(want).max()))


@pytest.mark.parametrize("M,N,K,splits", [(256, 256, 128, 2), (129, 300, 200, 3), (300, 1024, 4096, 4), (700, 6144, 1536, 3),
                                          (1, 8, 64, 4), (520, 264, 8 * 67, 2), (256, 520, 4096, 3)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_tcgen05_pair_product_with_k_split_over_a_cluster(M, N, K, splits, out_dtype):
    """K split over 2 to 4 pairs of one cluster, partial tiles summed over distributed shared memory: ragged
    edges in tokens, rows of W and K (a last K block that is partly beyond K, more K ranges than K blocks), in
    both output types; equal to the 64-bit product within the bound of the unsplit kernel, the same to the bit on
    a second run, and - with one key/row made to stand out in the LAST K range only - not blind to any range."""
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(M + 3 * N + K + splits)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    x[M // 2, K - 3] = 60.0                                   # one product that only the last K range sees
    w[N // 3, K - 3] = 50.0
    want = x.double() @ w.double().T
    out = torch.full((M, N), float("nan"), dtype=DT[out_dtype], device="cuda")
    ops.gemm_tcgen05_pair(x, w, out, splits=splits)
    assert ops.tcgen05_status("cuda") == 0, "a wait inside the kernel gave up"
    base, rel = (4e-5 * math.sqrt(K) * 4, 1e-6) if out_dtype == "float32" else (0.02 * math.sqrt(K), 2.0 ** -8)
    excess = ((out.double() - want).abs() - (base + rel * want.abs())).max().item()
    assert excess <= 0, f"an output is {excess:.3e} beyond its bound"
    assert abs(out[M // 2, N // 3].item() - want[M // 2, N // 3].item()) <= 16.0 and want[M // 2, N // 3].item() > 2000.0
    again = torch.full_like(out, float("nan"))
    ops.gemm_tcgen05_pair(x, w, again, splits=splits)
    assert torch.equal(out, again)
    with pytest.raises(ops.KernelError):
        ops.gemm_tcgen05_pair(x, w, out, splits=5)


@pytest.mark.parametrize("nq,nkv,d,K", [(4, 2, 128, 256), (3, 1, 64, 136), (2, 2, 256, 64), (8, 2, 128, 512)])
@pytest.mark.parametrize("with_norm,with_tables", [(True, True), (False, True), (True, False)])
def test_tcgen05_pair_product_with_the_qkv_epilogue(nq, nkv, d, K, with_norm, with_tables):
    """The q/k/v product with norm, rotation and cache write in its epilogue, for prompts of unequal lengths that
    continue sequences already in the cache (positions do not start at 0) over shuffled pages: q and the written
    keys and values agree with the plain float64 norm and rotation of the bfloat16-rounded product, and with the
    product + qkv_prepare pair of kernels to within one rounding; cache rows of other tokens are not touched; a layer
    that reads another layer's cache writes nothing."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(nq + d + K)
    eps, theta = 1e-5, 30000.0
    before, new = [0, 70, 5], [150, 9, 300]                   # tokens already cached, tokens of this step
    totals = [a + b for a, b in zip(before, new)]
    table, kp, vp = paged_case(rng, totals, nkv, d, "bfloat16")
    kp.fill_(7.0); vp.fill_(7.0)                              # a canary in every cell
    table_d = torch.as_tensor(table).cuda()
    seq = np.concatenate([np.full(n, s) for s, n in enumerate(new)]).astype(np.int32)
    pos = np.concatenate([np.arange(a, a + n) for a, n in zip(before, new)]).astype(np.int32)
    M = len(seq)
    seq_d, pos_d = torch.as_tensor(seq).cuda(), torch.as_tensor(pos).cuda()
    x = dev(rng.normal(0, 1, (M, K)), "bfloat16")
    w = dev(rng.normal(0, 1.0 / math.sqrt(K), ((nq + 2 * nkv) * d, K)), "bfloat16")
    qw = dev(1 + rng.normal(0, 0.1, d), "float32") if with_norm else None
    kw = dev(1 + rng.normal(0, 0.1, d), "float32") if with_norm else None
    cos, sin = plain.rope_table(max(totals), d, theta)
    cos_d, sin_d = (dev(cos, "float32"), dev(sin, "float32")) if with_tables else (None, None)
    q = torch.full((M, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05_pair_qkv(x, w, q, kp, vp, qw, kw, cos_d, sin_d, eps, seq_d, pos_d, table_d, M, nq, nkv, d)
    assert ops.tcgen05_status("cuda") == 0
    # the two-kernel path on a cache of its own
    kp2, vp2 = torch.full_like(kp, 7.0), torch.full_like(vp, 7.0)
    qkv = torch.empty(M, (nq + 2 * nkv) * d, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05_pair(x, w, qkv)
    q2 = torch.empty_like(q)
    ops.qkv_prepare(qkv, q2, kp2, vp2, qw, kw, cos_d, sin_d, seq_d, pos_d, table_d, M, nq, nkv, d, eps)
    # plain: norm and rotation of the rounded product
    raw = back(qkv).reshape(M, nq + 2 * nkv, d)
    rnd = plain.round_bf16
    qs, ks, vs = raw[:, :nq], raw[:, nq:nq + nkv], raw[:, nq + nkv:]
    if with_norm:
        qs, ks = plain.rms_norm(qs, back(qw), eps, rnd), plain.rms_norm(ks, back(kw), eps, rnd)
    if with_tables:
        qs, ks = plain.apply_rope(qs, pos, cos, sin, rnd), plain.apply_rope(ks, pos, cos, sin, rnd)
    scale = max(1.0, float(np.abs(qs).max()), float(np.abs(ks).max()))
    assert np.max(np.abs(back(q).reshape(M, nq, d) - qs)) <= 2.0 ** -7 * scale
    assert np.max(np.abs(back(q) - back(q2))) <= 2.0 ** -7 * scale
    written = torch.zeros(kp.shape[0], 64, dtype=torch.bool)
    for t in range(M):
        page, row = int(table[seq[t], pos[t] // 64]), int(pos[t] % 64)
        written[page, row] = True
        assert np.max(np.abs(back(kp[page, :, row]) - ks[t])) <= 2.0 ** -7 * scale, t
        assert np.array_equal(back(vp[page, :, row]), vs[t]), t
    touched = ((kp != 7.0) | (vp != 7.0)).any(dim=-1).any(dim=1).cpu()
    assert torch.equal(touched, written)
    assert np.max(np.abs(back(kp) - back(kp2))) <= 2.0 ** -7 * scale and torch.equal(vp, vp2)
    # a layer that reads another layer's cache
    kp3, vp3 = torch.full_like(kp, 7.0), torch.full_like(vp, 7.0)
    q3 = torch.empty_like(q)
    ops.gemm_tcgen05_pair_qkv(x, w, q3, kp3, vp3, qw, kw, cos_d, sin_d, eps, seq_d, pos_d, table_d, M, nq, nkv, d, write_kv=False)
    assert torch.equal(q3, q) and bool((kp3 == 7.0).all()) and bool((vp3 == 7.0).all())
    with pytest.raises(ops.KernelError):
        ops.gemm_tcgen05_pair_qkv(x, w[:, :K - 8].contiguous(), q3, kp3, vp3, qw, kw, cos_d, sin_d, eps, seq_d, pos_d, table_d,
                                  M, nq, nkv, d)


@pytest.mark.parametrize("M,inter,K,splits", [(300, 160, 192, 2), (512, 1536, 512, 3), (77, 112, 320, 4)])
def test_tcgen05_pair_gated_epilogue_with_k_split(M, inter, K, splits):
    """SiLU and gating after the partial tiles have met: equal to the split product + silu_mul, bit for bit."""
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(M + inter + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    gate = (torch.randn(inter, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    up = (torch.randn(inter, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate, up)
    fused = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05_pair(x, w, fused, gated=True, splits=splits)
    gate_up = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05_pair(x, w, gate_up, splits=splits)
    two = torch.empty_like(fused)
    ops.silu_mul(gate_up, two, interleaved=True)
    assert ops.tcgen05_status("cuda") == 0
    assert torch.equal(fused, two)
    gd = plain.round_bf16(back(x) @ back(gate).T)
    ud = plain.round_bf16(back(x) @ back(up).T)
    want = plain.silu_multiply(gd, ud, plain.round_bf16)
    assert np.max(np.abs(back(fused) - want)) <= 2e-2 * max(1.0, float(np.abs(want).max()))


@pytest.mark.parametrize("M,inter,K", [(128, 128, 64), (300, 160, 96), (2048, 1536, 512), (77, 112, 80)])
def test_tcgen05_prompt_gated_epilogue(M, inter, K):
    """The prompt kernel with SiLU and gating in its epilogue equals product + silu_mul, bit for bit."""
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(M + inter + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    gate = (torch.randn(inter, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    up = (torch.randn(inter, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate, up)
    fused = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05_prompt_gated(x, w, fused)
    gate_up = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tcgen05_prompt(x, w, gate_up)
    two = torch.empty_like(fused)
    ops.silu_mul(gate_up, two, interleaved=True)
    assert ops.tcgen05_status("cuda") == 0
    assert torch.equal(fused, two)
    gd = plain.round_bf16(back(x) @ back(gate).T)
    ud = plain.round_bf16(back(x) @ back(up).T)
    want = plain.silu_multiply(gd, ud, plain.round_bf16)
    assert np.max(np.abs(back(fused) - want)) <= 2e-2 * max(1.0, float(np.abs(want).max()))


@pytest.mark.parametrize("nq,nkv,d", [(8, 2, 128), (4, 4, 64), (6, 1, 128), (4, 2, 64)])
def test_prefill_attention_tcgen05_kernel(nq, nkv, d):
    """The TMA + tcgen05 attention: prompts of unequal length in one launch, then a second launch
    that continues them from the cache, over shuffled pages, against float64 causal attention.
    One sequence carries a score pattern that forces the running maximum to be raised late."""
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(nq * 17 + d)
    lengths, first = [700, 5, 129, 64, 333, 1000], [256, 1, 100, 63, 130, 999]
    table, kp, vp = paged_case(rng, lengths, nkv, d, "bfloat16")
    table_d = torch.as_tensor(table).cuda()
    full = [rng.normal(0, 1, (n, (nq + 2 * nkv) * d)) for n in lengths]
    # late keys with much larger scores than early ones: the accumulator has to be rescaled in TMEM
    full[0][600:, nq * d:(nq + nkv) * d] *= 6.0
    got = [np.zeros((n, nq * d)) for n in lengths]
    for part in range(2):
        spans = [(0, f) if part == 0 else (f, n) for f, n in zip(first, lengths)]
        rows = np.concatenate([full[s][a:b] for s, (a, b) in enumerate(spans)])
        seq = np.concatenate([np.full(b - a, s) for s, (a, b) in enumerate(spans)]).astype(np.int32)
        pos = np.concatenate([np.arange(a, b) for a, b in spans]).astype(np.int32)
        starts = np.cumsum([0] + [b - a for a, b in spans]).astype(np.int32)
        N = rows.shape[0]
        q = torch.empty(N, nq * d, dtype=torch.bfloat16, device="cuda")
        out = torch.zeros_like(q)
        seq_d, pos_d = torch.as_tensor(seq).cuda(), torch.as_tensor(pos).cuda()
        ops.qkv_prepare(dev(rows, "bfloat16"), q, kp, vp, None, None, None, None, seq_d, pos_d, table_d, N, nq, nkv, d, 0.0)
        ops.attention_prefill_tc(q, kp, vp, out, torch.as_tensor(starts).cuda(),
                                 torch.as_tensor([a for a, _ in spans], dtype=torch.int32).cuda(), table_d, len(lengths),
                                 max(b - a for a, b in spans), N, nq, nkv, d, d ** -0.5)
        assert ops.tcgen05_status("cuda") == 0, "a wait inside the kernel gave up"
        o = back(out)
        k = 0
        for s, (a, b) in enumerate(spans):
            got[s][a:b] = o[k:k + b - a]
            k += b - a
    for s, n in enumerate(lengths):
        x = stored(full[s], "bfloat16")
        qs = x[:, :nq * d].reshape(n, nq, d)
        ks = x[:, nq * d:(nq + nkv) * d].reshape(n, nkv, d)
        vs = x[:, (nq + nkv) * d:].reshape(n, nkv, d)
        want = plain.gqa_attention(qs, ks, vs).reshape(n, nq * d)
        err = np.abs(got[s] - want).max(axis=1)
        assert err.max() <= 2e-2, f"sequence {s}: row {int(err.argmax())} of {n}: max abs err {err.max():.3e}"
