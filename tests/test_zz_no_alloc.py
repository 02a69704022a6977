"""The allocation-free decode attention (csrc/attention_decode_static.h), called through its
exported C symbol as a host program without an allocator would call it, against the regular
entry point that takes the scratch buffer from its caller.  Collected last on purpose: a run
that stops at the first failure has then run every other test."""
import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

ERR_STATIC_SCRATCH = 10004
MAX_FLOATS = 2 * 1024 * 1024


def load_static(d):
    from qwen3_b200.csrc.build import compile_library
    lib = ctypes.CDLL(compile_library("attention_decode_static.cu", (f"Q3_HEAD_DIM={d}",)))
    fn = lib.q3_attention_decode_bf16_static
    fn.argtypes = [c_void_p] * 7 + [c_int, c_int64, c_int, c_int, c_float, c_int, c_int, c_void_p]
    fn.restype = c_int
    return fn


def make_case(seed, lengths, nq, nkv, d):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages_per_seq = max(-(-n // 64) for n in lengths)
    n_pages = sum(-(-n // 64) for n in lengths)
    order = torch.randperm(n_pages, generator=g, device="cuda").to(torch.int32)
    table = torch.full((len(lengths), pages_per_seq), -1, dtype=torch.int32, device="cuda")
    k = 0
    for s, n in enumerate(lengths):
        cnt = -(-n // 64)
        table[s, :cnt] = order[k:k + cnt]
        k += cnt
    kp = torch.randn(n_pages, nkv, 64, d, generator=g, device="cuda").to(torch.bfloat16)
    vp = torch.randn(n_pages, nkv, 64, d, generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn(len(lengths), nq * d, generator=g, device="cuda").to(torch.bfloat16)
    seq = torch.arange(len(lengths), dtype=torch.int32, device="cuda")
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
    return q, kp, vp, seq, pos, table


def plain_decode_attention(q, kp, vp, pos, table, nq, nkv, d):
    """float64 attention of one new token per sequence over its pages: the formulas of
    src/ops/gqa_attention.cu:84-153 (score = dot * d^-0.5, softmax, weighted sum / normaliser)."""
    q, kp, vp = q.double().cpu().numpy(), kp.double().cpu().numpy(), vp.double().cpu().numpy()
    pos, table = pos.cpu().numpy(), table.cpu().numpy()
    out = np.zeros((q.shape[0], nq * d))
    for t in range(q.shape[0]):
        n = int(pos[t]) + 1
        pages = table[t, : -(-n // 64)]
        for h in range(nq):
            keys = kp[pages, h // (nq // nkv)].reshape(-1, d)[:n]
            values = vp[pages, h // (nq // nkv)].reshape(-1, d)[:n]
            s = keys @ q[t, h * d:(h + 1) * d] * d ** -0.5
            w = np.exp(s - s.max())
            out[t, h * d:(h + 1) * d] = (w @ values) / w.sum()
    return out


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    from qwen3_b200.csrc import ops
    nq, nkv, d = 32, 8, 128
    fn = load_static(d)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different shapes and split counts: the second finds the first one's
    # leftovers in the shared array and must not care
    for turn, (seed, lengths, splits) in enumerate(((1, [700, 64, 1, 333], 5), (2, [130, 1000, 65], 3))):
        q, kp, vp, seq, pos, table = make_case(seed, lengths, nq, nkv, d)
        B = len(lengths)
        want = torch.zeros(B, nq * d, dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(B * nq * splits * (d + 2), dtype=torch.float32, device="cuda")
        ops.attention_decode(q, kp, vp, want, scratch, seq, pos, table, B, nq, nkv, d, d ** -0.5, None, splits)
        got = torch.zeros_like(want)
        torch.cuda.synchronize()
        # free device memory as the driver counts it: a cudaMalloc inside the library would show here,
        # which torch's own counters cannot see.  The first call on a device loads the module and sets a
        # kernel attribute, which may take memory once; from the second call on nothing may move.
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), got.data_ptr(), seq.data_ptr(), pos.data_ptr(),
                table.data_ptr(), table.shape[1], B, nq, nkv, d ** -0.5, 0, splits, stream)
        torch.cuda.synchronize()
        assert rc == 0
        if turn > 0:
            assert torch.cuda.mem_get_info()[0] == free_before
        # the same kernels on the same inputs: equal bit for bit
        assert torch.equal(got, want), f"max abs diff {(got.float() - want.float()).abs().max().item():.3e}"
        exact = plain_decode_attention(q, kp, vp, pos, table, nq, nkv, d)
        err = float(np.abs(got.double().cpu().numpy() - exact).max())
        assert err <= 1.5e-2, f"max abs err {err:.3e}"          # the tolerance of the kernel tests
        assert np.abs(exact).max() > 0.1


def test_static_scratch_entry_point_refuses_what_does_not_fit(capfd):
    nq, nkv, d = 32, 8, 128
    fn = load_static(d)
    q, kp, vp, seq, pos, table = make_case(3, [64], nq, nkv, d)
    out = torch.zeros(1, nq * d, dtype=torch.bfloat16, device="cuda")
    too_many = MAX_FLOATS // (nq * 32 * (d + 2)) + 1            # tokens that no longer fit with 32 splits
    rc = fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), out.data_ptr(), seq.data_ptr(), pos.data_ptr(),
            table.data_ptr(), table.shape[1], too_many, nq, nkv, d ** -0.5, 0, 32,
            torch.cuda.current_stream().cuda_stream)
    assert rc == ERR_STATIC_SCRATCH
    assert "built-in array holds" in capfd.readouterr().err
    # the largest sizes the argument checks let through are refused by the scratch check (its count cannot wrap),
    # and a split count beyond the launch limits is refused before it
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), out.data_ptr(), seq.data_ptr(), pos.data_ptr(),
            table.data_ptr(), table.shape[1], 65535, 16 * 65535, 65535, d ** -0.5, 0, 65535, stream)
    assert rc == ERR_STATIC_SCRATCH
    rc = fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), out.data_ptr(), seq.data_ptr(), pos.data_ptr(),
            table.data_ptr(), table.shape[1], 1, nq, nkv, d ** -0.5, 0, 70000, stream)
    assert rc == 10002
    torch.cuda.synchronize()
    assert out.float().abs().max().item() == 0.0                # nothing was launched
