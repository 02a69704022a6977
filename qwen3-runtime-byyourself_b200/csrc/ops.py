"""Python face of the CUDA entry points: tensors in, launches on torch's current stream.

Each function checks what the kernel relies on (device, dtype, contiguity, sizes),
passes raw pointers to the `extern "C"` entry point and raises `KernelError` if the
launch reports an error.  Nothing here computes on the host and nothing falls back
to a library: a CPU tensor or a missing compiler is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_uint64, c_void_p
from typing import Optional

import torch

from ..cache.book import PAGE_TOKENS
from .build import load_library

_ERRORS = {10001: "a size the kernel does not take", 10002: "more rows than one launch takes",
           10003: "a pointer or stride that is not 16-byte aligned"}
_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}
_fn_cache = {}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


# Programmatic dependent launch: a kernel launched with it may start (set up its barriers and tensor memory, fetch
# weights) while the kernel before it on the stream drains, and waits for that kernel's results only where it
# first needs them.  By default the sources named here launch their kernels that way: measured on whole decode
# steps of an 8B-sized model, the TMA + tcgen05 products gain 2.5-5 % at batches of 16 to 64 (4.92 -> 4.74 ms a
# step at batch 16), while the few-row product loses (batch 8: chains of waiting blocks take the room that a kernel's
# own later waves need) and the decode attention, which asks for its first pages before it waits, gains 0.5 % at batch
# 16 and 32 and loses 0.3 % at batch 64.  QWEN3_B200_PDL=1 / =0 turns it on / off for all.
PDL_SOURCES = ("gemm_tcgen05.cu",)
_pdl_override = {"1": True, "0": False}.get(os.environ.get("QWEN3_B200_PDL", ""))
_libs = {}


def _pdl_for(source: str) -> bool:
    return _pdl_override if _pdl_override is not None else source in PDL_SOURCES


def set_pdl(on) -> None:
    """Programmatic dependent launch for every kernel of the library (True / False), or back to the default
    (None): on for the sources in `PDL_SOURCES` only."""
    global _pdl_override
    _pdl_override = None if on is None else bool(on)
    for (source, _), lib in _libs.items():
        lib.q3_set_pdl(int(_pdl_for(source)))


class KernelTimer:
    """Times every launch of this library with a pair of CUDA events while it is active:

        with ops.KernelTimer() as timer:
            engine.step(...)
        timer.summary()  ->  {entry point: (launches, total microseconds)}

    For steps that are launched afresh (a captured step is one replay and shows nothing).  The events add a
    few microseconds of host work per launch, so the step as a whole runs slower than untimed; the
    durations are those of the kernels."""

    def __init__(self):
        self.records = []

    def __enter__(self):
        global _timer
        self._before, _timer = _timer, self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = self._before
        return False

    def run(self, name, fn, args):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream = torch.cuda.ExternalStream(_stream()) if _stream() else torch.cuda.current_stream()
        start.record(stream)
        code = fn(*args)
        stop.record(stream)
        self.records.append((name, start, stop))
        return code

    def summary(self) -> dict:
        torch.cuda.synchronize()
        out = {}
        for name, start, stop in self.records:
            n, us = out.get(name, (0, 0.0))
            out[name] = (n + 1, us + start.elapsed_time(stop) * 1e3)
        return out


_timer: Optional[KernelTimer] = None


def _fn(source: str, name: str, argtypes, defines=()):
    fn = _fn_untimed(source, name, argtypes, defines)
    if _timer is None:
        return fn
    timer = _timer
    return lambda *args: timer.run(name, fn, args)


def _fn_untimed(source: str, name: str, argtypes, defines=()):
    key = (source, name, tuple(defines))
    fn = _fn_cache.get(key)
    if fn is None:
        lib = load_library(source, defines)
        if (source, tuple(defines)) not in _libs:
            _libs[(source, tuple(defines))] = lib
            lib.q3_set_pdl.argtypes = [c_int]
            lib.q3_set_pdl.restype = None
            lib.q3_set_pdl(int(_pdl_for(source)))
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _fn_cache[key] = fn
    return fn


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched (or captured into a graph) so far."""
    return _launches


def _count_extra(n: int) -> None:
    """Entry points that launch more than one kernel add the rest here."""
    global _launches
    _launches += n


def _check(code: int, name: str):
    global _launches
    _launches += 1
    if code != 0:
        what = _ERRORS.get(code)
        if what is None:
            what = f"CUDA error {code} at launch"
        raise KernelError(f"{name}: {what}")


_pinned_stream: Optional[int] = None


def _stream() -> int:
    return _pinned_stream if _pinned_stream is not None else torch.cuda.current_stream().cuda_stream


class on_current_stream:
    """Within this scope every launch goes to the stream that is current on entry, looked up once
    (asking torch for the current stream costs more than a launch)."""

    def __enter__(self):
        global _pinned_stream
        self._before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self._before
        return False


def _dev(t: torch.Tensor, name: str, dtype=None):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t.data_ptr()


def _suffix(t: torch.Tensor) -> str:
    try:
        return _SUFFIX[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor], name: str, dtype=None):
    return None if t is None else _dev(t, name, dtype)


# ------------------------------------------------------------------ elementwise
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]]; ids int32 [N], table [V, H], out [N, H]."""
    s = _suffix(table)
    fn = _fn("elementwise.cu", f"q3_embedding_{s}", [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    n = ids.numel()
    if out.shape[0] < n or out.shape[1] != table.shape[1] or out.dtype != table.dtype:
        raise KernelError("embedding: output does not fit")
    _check(fn(_dev(ids, "ids", torch.int32), _dev(table, "table"), _dev(out, "out"), n, table.shape[1],
              table.shape[0], _stream()), "embedding")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             delta: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = RMSNorm(x) * weight over the last dimension; weight is float32.

    With `delta`, first x += delta in place (32-bit sum, stored in x's type) and the
    norm reads the stored sum.  x: [..., size] with contiguous rows."""
    s = _suffix(x)
    size = x.shape[-1]
    rows = x.numel() // size if size else 0
    if weight.numel() != size or out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("rms_norm: weight or output does not fit")
    if delta is not None and (delta.shape != x.shape or delta.dtype != x.dtype):
        raise KernelError("rms_norm: delta does not fit")
    if out.data_ptr() == x.data_ptr():
        raise KernelError("rms_norm: the output may not be the input's own memory")
    fn = _fn("elementwise.cu", f"q3_rms_norm_{s}",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_int64, c_int64, c_void_p])
    _check(fn(_dev(x, "x"), _ptr(delta, "delta"), _dev(weight, "weight", torch.float32), _dev(out, "out"),
              rows, size, float(eps), size, size, _stream()), "rms_norm")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """out[r, c] = silu(gate[r, c]) * up[r, c]; a row of `gate_up` holds the gate in its first half
    and the up values in its second, or (`interleaved`) blocks of eight gate columns each followed
    by the eight up columns of the same features."""
    s = _suffix(gate_up)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("silu_mul: output does not fit")
    fn = _fn("elementwise.cu", f"q3_silu_mul_{s}", [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    _check(fn(_dev(gate_up, "gate_up"), _dev(out, "out"), rows, two_i // 2, int(bool(interleaved)), _stream()),
           "silu_mul")
    return out


def gather_rows(x: torch.Tensor, idx: torch.Tensor, out: torch.Tensor, delta: Optional[torch.Tensor] = None):
    """out[r] = x[idx[r]] (+ delta[idx[r]], summed in 32-bit)."""
    s = _suffix(x)
    rows, size = idx.numel(), x.shape[-1]
    if out.shape[0] < rows or out.shape[-1] != size or out.dtype != x.dtype:
        raise KernelError("gather_rows: output does not fit")
    fn = _fn("elementwise.cu", f"q3_gather_rows_{s}", [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p])
    _check(fn(_dev(x, "x"), _ptr(delta, "delta", x.dtype), _dev(idx, "idx", torch.int32), _dev(out, "out"),
              rows, size, _stream()), "gather_rows")
    return out


def place_rows(src: torch.Tensor, dst: torch.Tensor, block_rows: int = 0, dst_block_stride: int = 0, dst_row0: int = 0):
    """Rows of `src` [rows, cols] into `dst` [*, cols], converted to dst's type on the way: source row r goes to
    row dst_row0 + (r // block_rows) * dst_block_stride + r % block_rows (block_rows 0: one block, consecutive
    rows from dst_row0).  Load time: the q, k and v matrices into one, gate and up rows interleaved."""
    kinds = {torch.float32: 0, torch.bfloat16: 1}
    if src.dtype not in kinds or dst.dtype not in kinds:
        raise KernelError("place_rows: float32 or bfloat16 on either side")
    rows, cols = src.shape
    block = int(block_rows) or rows
    stride = int(dst_block_stride) or block
    if dst.shape[-1] != cols or rows % block != 0:
        raise KernelError("place_rows: shapes do not fit")
    last = dst_row0 + (rows // block - 1) * stride + block if rows else 0
    if last > dst.shape[0]:
        raise KernelError("place_rows: the rows do not fit the destination")
    fn = _fn("elementwise.cu", "q3_place_rows", [c_void_p, c_int, c_void_p, c_int] + [c_int64] * 5 + [c_void_p])
    _check(fn(_dev(src, "src"), kinds[src.dtype], _dev(dst, "dst"), kinds[dst.dtype], rows, cols, block, stride, int(dst_row0),
              _stream()), "place_rows")
    return dst


# ------------------------------------------------------------------ matrix products
def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T in true 32-bit (fmaf, fixed order over K)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_f32.cu", "q3_gemm_tn_f32",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_void_p])
    _check(fn(_dev(x, "x", torch.float32), _dev(w, "w", torch.float32), _dev(out, "out", torch.float32),
              M, N, K, K, K, N, _stream()), "gemm_f32")
    return out


def gemm_bf16_any_width(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for bfloat16 operands of any width K, on the CUDA cores with 32-bit
    accumulation: the product for widths that the tensor-core kernels refuse (K no multiple of 8)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_bf16_any_width: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_f32.cu", "q3_gemm_tn_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K, K, K, N,
              int(out.dtype == torch.float32), _stream()), "gemm_bf16_any_width")
    return out


# ------------------------------------------------------------------ attention
def _rotary_dim(cos, sin, d: int) -> int:
    """How many leading values of a head the tables rotate: twice their width (the head size without tables)."""
    if cos is None:
        return d
    if sin is None or cos.shape != sin.shape or cos.dim() != 2 or 2 * cos.shape[1] > d:
        raise KernelError("rotation tables are [positions, rotary_dim / 2] with rotary_dim <= head_dim")
    return 2 * cos.shape[1]


def qkv_prepare(qkv, q_out, k_pages, v_pages, q_norm_w, k_norm_w, cos, sin, token_seq, token_pos, page_table,
                n_tokens: int, nq: int, nkv: int, d: int, eps: float, write_kv: bool = True):
    """Per-head norm of q and k, rotation, and the write of k and v into the cache pages
    (`write_kv=False`: only q is prepared, for a layer that reads another layer's cache)."""
    s = _suffix(qkv)
    if d % 16 != 0 or d > 256:
        raise KernelError(f"head_dim {d} is not supported: multiples of 16 up to 256")
    if qkv.shape[-1] != (nq + 2 * nkv) * d or k_pages.dtype != qkv.dtype or k_pages.shape[1:] != (nkv, PAGE_TOKENS, d):
        raise KernelError("qkv_prepare: shapes do not fit")
    rot = _rotary_dim(cos, sin, d)
    fn = _fn("attention.cu", f"q3_qkv_prepare_{s}",
             [c_void_p] * 11 + [c_int, c_int64, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p])
    _check(fn(_dev(qkv, "qkv"), _dev(q_out, "q_out", qkv.dtype), _dev(k_pages, "k_pages"), _dev(v_pages, "v_pages"),
              _ptr(q_norm_w, "q_norm_w", torch.float32), _ptr(k_norm_w, "k_norm_w", torch.float32),
              _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], n_tokens, nq, nkv, d, float(eps),
              int(bool(write_kv)), rot, _stream()), "qkv_prepare")
    return q_out


def attention_generic(q, k_pages, v_pages, out, token_seq, token_pos, page_table, n_tokens: int, nq: int, nkv: int,
                      d: int, scale: float, window: Optional[int] = None):
    """Causal grouped-query attention of every token of the step over its sequence's pages."""
    s = _suffix(q)
    if d % 16 != 0 or d > 256:
        raise KernelError(f"head_dim {d} is not supported: multiples of 16 up to 256")
    fn = _fn("attention.cu", f"q3_attention_generic_{s}",
             [c_void_p] * 7 + [c_int, c_int64, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", q.dtype), _dev(v_pages, "v_pages", q.dtype),
              _dev(out, "out", q.dtype), _dev(token_seq, "token_seq", torch.int32),
              _dev(token_pos, "token_pos", torch.int32), _dev(page_table, "page_table", torch.int32),
              page_table.shape[-1], n_tokens, nq, nkv, d, float(scale), int(window or 0), _stream()),
           "attention_generic")
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor, valid: Optional[int] = None) -> torch.Tensor:
    """out[r] = index of the highest logit of row r (lowest id among equals, NaN as -inf)."""
    rows, vocab = logits.shape
    fn = _fn("sampling.cu", "q3_argmax_f32", [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(logits, "logits", torch.float32), vocab, rows, int(valid or vocab),
              _dev(out, "out", torch.int32), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int,
           seq_ids: torch.Tensor, steps, valid: Optional[int] = None) -> torch.Tensor:
    """One draw per row; out[r] = -1 marks a row with a non-finite logit.  `steps` is an int32 tensor with
    the step of every row, or one int for all rows."""
    rows, vocab = logits.shape
    fn = _fn("sampling.cu", "q3_sample_f32",
             [c_void_p, c_int64, c_int, c_int, c_float, c_int, c_float, c_uint64, c_void_p, c_void_p, c_int, c_void_p,
              c_void_p])
    per_row = isinstance(steps, torch.Tensor)
    _check(fn(_dev(logits, "logits", torch.float32), vocab, rows, int(valid or vocab), float(temperature), int(top_k),
              float(top_p), int(seed) & 0xFFFFFFFFFFFFFFFF, _dev(seq_ids, "seq_ids", torch.int64),
              _dev(steps, "steps", torch.int32) if per_row else None, 0 if per_row else int(steps),
              _dev(out, "out", torch.int32), _stream()), "sample")
    return out


# ------------------------------------------------------------------ bfloat16 decode attention
def attention_decode_splits(n_tokens: int, nkv: int, sm_count: int) -> int:
    """Key splits such that the whole grid (splits x kv heads x tokens) is resident at once, two
    blocks per SM, and at most 16: fixed by the batch size alone.  (Measured at batch 8, 4,096
    keys: 4 splits 29 us, 5 splits - a second wave - 39 us.)"""
    return max(1, min(16, (2 * sm_count) // max(1, n_tokens * nkv)))


def attention_decode(q, k_pages, v_pages, out, scratch, token_seq, token_pos, page_table, n_tokens: int, nq: int,
                     nkv: int, d: int, scale: float, window: Optional[int], n_splits: int):
    """One token per sequence against its cached keys; `scratch` is float32 with at least
    n_tokens * nq * n_splits * (d + 2) elements."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode is a bfloat16 kernel")
    if nq // nkv > 16 or d % 16 != 0 or d > 256:
        raise KernelError(f"attention_decode: group of {nq // nkv} heads or head_dim {d} not supported")
    if scratch.numel() < n_tokens * nq * n_splits * (d + 2):
        raise KernelError("attention_decode: scratch too small")
    fn = _fn("attention_decode.cu", "q3_attention_decode_bf16",
             [c_void_p] * 8 + [c_int, c_int64, c_int, c_int, c_float, c_int, c_int, c_void_p],
             defines=(f"Q3_HEAD_DIM={d}",))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _dev(scratch, "scratch", torch.float32),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], n_tokens, nq, nkv, float(scale),
              int(window or 0), int(n_splits), _stream()), "attention_decode")
    _count_extra(1)
    return out


FUSED_DECODE_MAX_SPLITS = 16
_fused_max_splits = {}


def attention_decode_fused_max_splits(d: int, device) -> int:
    """The most key splits `attention_decode_fused` takes on `device` for head size `d`: 16 where the device places
    clusters of 16 blocks (beyond the portable size), else 8."""
    key = (d, torch.device(device))
    got = _fused_max_splits.get(key)
    if got is None:
        fn = _fn_untimed("attention_decode.cu", "q3_attention_decode_fused_max_splits", [], defines=(f"Q3_HEAD_DIM={d}",))
        with torch.cuda.device(key[1]):
            got = _fused_max_splits[key] = int(fn())
    return got


def attention_decode_fused(qkv, k_pages, v_pages, out, q_norm_w, k_norm_w, cos, sin, eps: float, token_seq, token_pos,
                           page_table, n_tokens: int, nq: int, nkv: int, d: int, scale: float, window: Optional[int],
                           n_splits: int, write_kv: bool = True):
    """The attention of a decode step in one launch: per-head norm and rotation of the new query and key, the
    write of key and value into the cache pages, attention over the pages split over the keys, and the merge of
    the splits inside a thread-block cluster.  `qkv` is the projection output [tokens, (nq + 2 nkv) * d]."""
    if qkv.dtype != torch.bfloat16:
        raise KernelError("attention_decode_fused is a bfloat16 kernel")
    if nq // nkv > 16 or d % 16 != 0 or d > 256 or not 0 < n_splits <= FUSED_DECODE_MAX_SPLITS:
        raise KernelError(f"attention_decode_fused: group of {nq // nkv} heads, head_dim {d} or {n_splits} splits not supported")
    if qkv.shape[-1] != (nq + 2 * nkv) * d or k_pages.shape[1:] != (nkv, PAGE_TOKENS, d) or out.shape[-1] != nq * d:
        raise KernelError("attention_decode_fused: shapes do not fit")
    fn = _fn("attention_decode.cu", "q3_attention_decode_fused_bf16",
             [c_void_p] * 8 + [c_float] + [c_void_p] * 3 + [c_int, c_int64, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
                                                            c_void_p],
             defines=(f"Q3_HEAD_DIM={d}",))
    _check(fn(_dev(qkv, "qkv"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _ptr(q_norm_w, "q_norm_w", torch.float32), _ptr(k_norm_w, "k_norm_w", torch.float32),
              _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32), float(eps),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], n_tokens, nq, nkv, float(scale),
              int(window or 0), int(n_splits), int(bool(write_kv)), _rotary_dim(cos, sin, d), _stream()), "attention_decode_fused")
    return out


# ------------------------------------------------------------------ bfloat16 weight-streaming product
SKINNY_MAX_ROWS = 64


def gemm_skinny_fits(M: int, K: int) -> bool:
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 64, bfloat16 operands, out bfloat16 or float32."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or not gemm_skinny_fits(M, K):
        raise KernelError(f"gemm_skinny: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    name = {torch.bfloat16: "q3_gemm_skinny_bf16", torch.float32: "q3_gemm_skinny_bf16_f32out"}.get(out.dtype)
    if name is None:
        raise KernelError("gemm_skinny: output must be bfloat16 or float32")
    fn = _fn("gemm_skinny_bf16.cu", name, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K, _stream()),
           "gemm_skinny")
    return out


# ------------------------------------------------------------------ bfloat16 prompt attention
def attention_prefill(q, k_pages, v_pages, out, seq_start, seq_pos0, page_table, n_seqs: int, max_new: int, nq: int,
                      nkv: int, d: int, scale: float, window: Optional[int] = None):
    """Causal attention of every new token of every sequence over its pages (tiled, tensor cores)."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill is a bfloat16 kernel")
    if d % 16 != 0 or d > 256:
        raise KernelError(f"head_dim {d} is not supported: multiples of 16 up to 256")
    fn = _fn("attention_prefill.cu", "q3_attention_prefill_bf16",
             [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
             defines=(f"Q3_HEAD_DIM={d}",))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_pos0, "seq_pos0", torch.int32), _dev(page_table, "page_table", torch.int32),
              page_table.shape[-1], n_seqs, max_new, nq, nkv, float(scale), int(window or 0), _stream()),
           "attention_prefill")
    return out


# ------------------------------------------------------------------ bfloat16 tcgen05 product
_tc_status = {}


def _status_word(device) -> torch.Tensor:
    word = _tc_status.get(device)
    if word is None:
        word = _tc_status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return word


def tcgen05_status(device) -> int:
    """0, or where a bounded wait inside the tcgen05 product gave up (1 producer, 2 MMA, 3 epilogue);
    reading it synchronises the device and clears it."""
    word = _status_word(torch.device(device))
    value = int(word.item())
    if value:
        word.zero_()
    return value


def gemm_tcgen05_mid(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: int = 0) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for a few hundred rows at most on the 5th-generation tensor cores,
    weights first: TMA-fed tiles of 128 rows of w, accumulator in tensor memory, K split over the `splits` blocks
    of a cluster (0 = chosen from N and K) that add their partial tiles through distributed shared
    memory.  bfloat16 operands, out bfloat16 or float32; K a multiple of 8."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or K % 8 != 0:
        raise KernelError(f"gemm_tcgen05_mid: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05_mid: output must be bfloat16 or float32")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_mid_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K,
              int(out.dtype == torch.float32), 0, int(splits), _status_word(x.device).data_ptr(), _stream()),
           "gemm_tcgen05_mid")
    return out


def gemm_tcgen05_mid_splits(M: int, N: int, K: int) -> int:
    """The number of K ranges `gemm_tcgen05_mid` chooses for this shape."""
    lib = load_library("gemm_tcgen05.cu", ())
    lib.q3_gemm_tcgen05_mid_splits.argtypes = [c_int, c_int, c_int]
    lib.q3_gemm_tcgen05_mid_splits.restype = c_int
    return int(lib.q3_gemm_tcgen05_mid_splits(N, K, M))


def gemm_tcgen05_mid_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: int = 0) -> torch.Tensor:
    """out[M, N/2] = round(silu(g)) * u for a few hundred rows at most; `w` [N, K] holds the gate and up rows interleaved
    in blocks of eight (`interleave_gate_up`); the gating runs where the cluster's partial tiles are added."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2) or K % 8 != 0 or N % 16 != 0 or out.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05_mid_gated: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_mid_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K, 0, 1, int(splits),
              _status_word(x.device).data_ptr(), _stream()), "gemm_tcgen05_mid_gated")
    return out


def gemm_skinny_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N/2] = round(silu(g)) * u where g and u are the products of x with the gate and up rows of
    w [N, K], which holds them interleaved in blocks of eight rows (see `interleave_gate_up`)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2) or N % 16 != 0 or not gemm_skinny_fits(M, K):
        raise KernelError(f"gemm_skinny_gated: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_skinny_bf16.cu", "q3_gemm_skinny_gated_bf16", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out", torch.bfloat16), M, N, K,
              _stream()), "gemm_skinny_gated")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2I, K]: rows 16t..16t+7 are gate rows 8t..8t+7, rows 16t+8..16t+15 the up rows of the same features."""
    I, K = gate.shape
    if I % 8 != 0 or up.shape != gate.shape:
        raise KernelError("interleave_gate_up: the intermediate size must be a multiple of 8")
    return torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


def gemm_tcgen05_prompt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_n: int = 256) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for many rows: persistent blocks, tiles of 128 tokens by `tile_n`
    (128 or 256) rows of w, accumulators double-buffered in tensor memory."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or K % 8 != 0:
        raise KernelError(f"gemm_tcgen05_prompt: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05_prompt: output must be bfloat16 or float32")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_prompt_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K,
              int(out.dtype == torch.float32), int(tile_n), _status_word(x.device).data_ptr(), _stream()),
           "gemm_tcgen05_prompt")
    return out


def gemm_tcgen05_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False,
                      splits: int = 1) -> torch.Tensor:
    """The prompt product on pairs of SMs (tcgen05 cta_group::2): tiles of 256 tokens by 256 rows of w, each
    block of a pair loading its own tokens and half of the w tile.  `gated`: w holds gate and up rows
    interleaved in blocks of eight and out is [M, N/2] = round(silu(g)) * u.  `splits` (1..4): K split over
    that many pairs of one cluster, whose partial tiles are summed over distributed shared memory in a fixed
    order (for shapes with too few tiles, or a tile count just above a whole number of waves)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2 if gated else N) or K % 8 != 0 or (gated and N % 16 != 0):
        raise KernelError(f"gemm_tcgen05_pair: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if out.dtype not in ((torch.bfloat16,) if gated else (torch.bfloat16, torch.float32)):
        raise KernelError("gemm_tcgen05_pair: output must be bfloat16 (or float32 when not gated)")
    if not 1 <= splits <= PAIR_MAX_SPLITS:
        raise KernelError(f"gemm_tcgen05_pair: 1 to {PAIR_MAX_SPLITS} K ranges, not {splits}")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_pair_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K,
              int(out.dtype == torch.float32), int(gated), int(splits), _status_word(x.device).data_ptr(), _stream()),
           "gemm_tcgen05_pair")
    return out


PAIR_MAX_SPLITS = 4


def gemm_tcgen05_pair_capacity(splits: int) -> int:
    """How many pairs of SMs of the current device run at once when a cluster is `splits` pairs (0: none fit)."""
    fn = _fn_untimed("gemm_tcgen05.cu", "q3_gemm_tcgen05_pair_capacity", [c_int])
    return int(fn(int(splits)))


PAIR_QKV_HEAD_DIMS = (64, 128, 256)


def gemm_tcgen05_pair_qkv(x: torch.Tensor, w: torch.Tensor, q_out, k_pages, v_pages, q_norm_w, k_norm_w, cos, sin, eps,
                          token_seq, token_pos, page_table, n_tokens: int, nq: int, nkv: int, d: int,
                          write_kv: bool = True) -> None:
    """The q/k/v product of a prompt step on pairs of SMs with `qkv_prepare`'s work in its epilogue: per-head
    RMSNorm of q and k (weights may be None), rotation of the whole head (tables [positions, d/2], may be None),
    q into q_out [n_tokens, nq*d], k and v into the pages at the tokens' positions (`write_kv`); the product's
    own output is never stored.  w [(nq + 2 nkv) d, K] holds the q, k and v rows one after the other.  bfloat16,
    head sizes 64, 128 and 256."""
    M, K = x.shape
    if x.dtype != torch.bfloat16 or M != n_tokens or w.shape != ((nq + 2 * nkv) * d, K) or K % 8 != 0 or d not in PAIR_QKV_HEAD_DIMS:
        raise KernelError(f"gemm_tcgen05_pair_qkv: shapes {tuple(x.shape)} x {tuple(w.shape)}^T for {nq}+2*{nkv} heads of {d}")
    if q_out.shape != (n_tokens, nq * d) or (q_norm_w is None) != (k_norm_w is None) or (cos is None) != (sin is None):
        raise KernelError("gemm_tcgen05_pair_qkv: q_out, norm weights or tables do not fit")
    if cos is not None and _rotary_dim(cos, sin, d) != d:
        raise KernelError("gemm_tcgen05_pair_qkv rotates the whole head only")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_pair_qkv_bf16",
             [c_void_p, c_void_p, c_int, c_int] + [c_void_p] * 7 + [c_float] + [c_void_p] * 3 + [c_int] * 5 + [c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), M, K, _dev(q_out, "q_out", torch.bfloat16),
              _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _ptr(q_norm_w, "q_norm_w", torch.float32), _ptr(k_norm_w, "k_norm_w", torch.float32),
              _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32), float(eps),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], nq, nkv, d, int(bool(write_kv)),
              _status_word(x.device).data_ptr(), _stream()), "gemm_tcgen05_pair_qkv")


def gemm_tcgen05_prompt_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N/2] = round(silu(g)) * u for many rows; `w` [N, K] holds the gate and up rows interleaved in
    blocks of eight (`interleave_gate_up`); the gating runs in the product's epilogue."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2) or K % 8 != 0 or N % 16 != 0 or out.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05_prompt_gated: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_prompt_gated_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K,
              _status_word(x.device).data_ptr(), _stream()), "gemm_tcgen05_prompt_gated")
    return out


# ------------------------------------------------------------------ bfloat16 prompt attention on tcgen05
def attention_prefill_tc_fits(d: int, window: Optional[int]) -> bool:
    return d in (64, 128) and not window


def attention_prefill_tc(q, k_pages, v_pages, out, seq_start, seq_pos0, page_table, n_seqs: int, max_new: int,
                         n_tokens: int, nq: int, nkv: int, d: int, scale: float):
    """Causal attention of every new token over its pages with both products on tcgen05 (TMA-fed,
    scores and output accumulated in tensor memory).  Head sizes 64 and 128."""
    if q.dtype != torch.bfloat16 or not attention_prefill_tc_fits(d, None):
        raise KernelError("attention_prefill_tc: bfloat16, head size 64 or 128")
    fn = _fn("attention_prefill_tc.cu", "q3_attention_prefill_tc_bf16",
             [c_void_p] * 7 + [c_int, c_int, c_int, c_int64, c_int64, c_int, c_int, c_float, c_void_p, c_void_p],
             defines=(f"Q3_HEAD_DIM={d}",))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_pos0, "seq_pos0", torch.int32), _dev(page_table, "page_table", torch.int32),
              page_table.shape[-1], n_seqs, max_new, n_tokens, k_pages.shape[0], nq, nkv, float(scale),
              _status_word(q.device).data_ptr(), _stream()), "attention_prefill_tc")
    return out
