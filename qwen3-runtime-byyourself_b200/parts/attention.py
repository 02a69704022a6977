"""Grouped-query attention over the paged cache, as a mixer part.

Order of operations as in the reference (src/model/self_attention.cpp:122-169):
q/k/v projections -> per-head RMSNorm of q and k -> rotation -> cache write ->
causal attention over the cache (scale d^-0.5 after the dot, 32-bit softmax) ->
output projection.  The three projections run as one product over the row-wise
concatenation [Wq; Wk; Wv] made at bind time; norm, rotation and the cache write are
one kernel.  Head counts, head size, scale, window, norm and position encoding are
parameters; the part does not know its model.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.book import CacheNeed
from ..config.plan import PartSpec
from ..csrc import ops
from ..weights.loader import WeightSpec
from ..weights.upload import fuse_rows
from .base import Part, build_part, register_part
from .linear import linear

# Hand-written bfloat16 kernels register themselves here: fn(part, q, cache, out, ctx, table) -> bool
PREFILL_KERNELS = []
DECODE_KERNELS = []
# Kernels that take the projection output as it is and do norm, rotation, cache write and attention of a decode
# step in one launch: fn(part, qkv, cache, out, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool
FUSED_DECODE_KERNELS = []
# Kernels that do the q/k/v product of a prompt step themselves, with norm, rotation and cache write in its
# epilogue: fn(part, x, cache, q, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool (q is filled, the pages written)
FUSED_PROJECTION_KERNELS = []


class GQAAttention(Part):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 qk_norm: Optional[PartSpec] = None, position: Optional[PartSpec] = None,
                 window: Optional[int] = None, prefix: str = ""):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 up to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale, self.window, self.prefix = float(scale), window, prefix
        self.q_norm = build_part("norm", qk_norm) if qk_norm else None
        self.k_norm = build_part("norm", qk_norm) if qk_norm else None
        self.position = build_part("position", position) if position else None
        self.w_qkv = self.w_o = None

    # -- weights
    def weight_specs(self, prefix: str) -> dict:
        p = prefix + self.prefix
        nq, nkv, d, H = self.num_heads, self.num_kv_heads, self.head_dim, self.hidden_size
        specs = {p + "q_proj.weight": WeightSpec((nq * d, H)), p + "k_proj.weight": WeightSpec((nkv * d, H)),
                 p + "v_proj.weight": WeightSpec((nkv * d, H)), p + "o_proj.weight": WeightSpec((H, nq * d))}
        if self.q_norm is not None:
            specs.update(self.q_norm.weight_specs(p + "q_norm.weight"))
            specs.update(self.k_norm.weight_specs(p + "k_norm.weight"))
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p = prefix + self.prefix
        self.w_qkv = fuse_rows(weights, [p + "q_proj.weight", p + "k_proj.weight", p + "v_proj.weight"])
        self.w_o = weights.pop(p + "o_proj.weight").contiguous()
        if self.q_norm is not None:
            self.q_norm.bind(weights, p + "q_norm.weight", dtype, device)
            self.k_norm.bind(weights, p + "k_norm.weight", dtype, device)

    # -- cache
    def cache_need(self) -> CacheNeed:
        return CacheNeed("window" if self.window else "full", self.num_kv_heads, self.head_dim, self.window)

    # -- step
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        N = ctx.n_tokens
        table = ctx.page_tables[cache.group]
        attn = ctx.scratch.get("attn.ctx", (N, nq * d), ctx.dtype)
        out = ctx.scratch.get("mixer.out", (N, self.hidden_size), ctx.dtype)
        norm_eps = self.q_norm.eps if self.q_norm is not None else 0.0
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        tables = self.position is None or getattr(self.position, "fused_tables", False)
        cos = sin = None
        if tables and self.position is not None:
            self.position.prepare(ctx.max_positions, ctx.device)
            cos, sin = self.position.cos, self.position.sin
        if tables and not ctx.is_decode and ctx.dtype == torch.bfloat16:
            q = ctx.scratch.get("attn.q", (N, nq * d), ctx.dtype)
            for kernel in FUSED_PROJECTION_KERNELS:
                if kernel(self, x, cache, q, ctx, table, qw, kw, norm_eps, cos, sin):
                    self.attend(q, cache, attn, ctx, table)
                    return linear(attn, self.w_o, out)
        qkv = ctx.scratch.get("attn.qkv", (N, (nq + 2 * nkv) * d), ctx.dtype)
        linear(x, self.w_qkv, qkv)
        if tables and ctx.is_decode and ctx.dtype == torch.bfloat16:
            for kernel in FUSED_DECODE_KERNELS:
                if kernel(self, qkv, cache, attn, ctx, table, qw, kw, norm_eps, cos, sin):
                    return linear(attn, self.w_o, out)
        q = ctx.scratch.get("attn.q", (N, nq * d), ctx.dtype)
        if tables:
            ops.qkv_prepare(qkv, q, cache.keys, cache.values, qw, kw, cos, sin, ctx.token_seq, ctx.token_pos, table,
                            N, nq, nkv, d, norm_eps, write_kv=not cache.shared)
        else:
            self._prepare_unfused(qkv, q, cache, ctx, table, qw, kw, norm_eps)
        self.attend(q, cache, attn, ctx, table)
        return linear(attn, self.w_o, out)

    def attend(self, q, cache, out, ctx, table) -> None:
        if ctx.dtype == torch.bfloat16:
            for kernel in (DECODE_KERNELS if ctx.is_decode else PREFILL_KERNELS):
                if kernel(self, q, cache, out, ctx, table):
                    return
        ops.attention_generic(q, cache.keys, cache.values, out, ctx.token_seq, ctx.token_pos, table, ctx.n_tokens,
                              self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window)

    def _prepare_unfused(self, qkv, q, cache, ctx, table, qw, kw, eps) -> None:
        """A position encoding without kernel tables: norm, then `apply_`, then the cache write."""
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        N = ctx.n_tokens
        qs = qkv[:, :nq * d].contiguous().view(N, nq, d)
        ks = qkv[:, nq * d:(nq + nkv) * d].contiguous().view(N, nkv, d)
        if qw is not None:                                  # into buffers of their own: the norm kernel's input and
            qn, kn = torch.empty_like(qs), torch.empty_like(ks)   # output may not be the same memory
            ops.rms_norm(qs, qw, eps, qn)
            ops.rms_norm(ks, kw, eps, kn)
            qs, ks = qn, kn
        self.position.prepare(ctx.max_positions, ctx.device)
        self.position.apply_(qs, ks, ctx.token_pos[:N])
        packed = torch.cat([qs.view(N, -1), ks.view(N, -1), qkv[:, (nq + nkv) * d:]], dim=1).contiguous()
        ops.qkv_prepare(packed, q, cache.keys, cache.values, None, None, None, None, ctx.token_seq, ctx.token_pos,
                        table, N, nq, nkv, d, 0.0, write_kv=not cache.shared)


def _decode_split_kernel(part, q, cache, out, ctx, table) -> bool:
    """The split-key tensor-core decode kernel: bfloat16, groups of up to 16 query heads."""
    nq, nkv, d = part.num_heads, part.num_kv_heads, part.head_dim
    if nq // nkv > 16:
        return False
    splits = ops.attention_decode_splits(ctx.n_tokens, nkv, _sm_count(ctx.device))
    scratch = ctx.scratch.get("attn.decode_scratch", (ctx.n_tokens * nq * splits * (d + 2),), torch.float32)
    ops.attention_decode(q, cache.keys, cache.values, out, scratch, ctx.token_seq, ctx.token_pos, table, ctx.n_tokens,
                         nq, nkv, d, part.scale, part.window, splits)
    return True


def _decode_fused_kernel(part, qkv, cache, out, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool:
    """Norm, rotation, cache write, split-key attention and the merge of the splits (inside a thread-block
    cluster) in one launch: bfloat16, groups of up to 16 query heads, up to 16 splits."""
    nq, nkv, d = part.num_heads, part.num_kv_heads, part.head_dim
    if nq // nkv > 16:
        return False
    splits = ops.attention_decode_splits(ctx.n_tokens, nkv, _sm_count(ctx.device))
    if splits > 8:
        # more than eight blocks per (sequence, kv head) - a cluster beyond the portable size - pay for one or two
        # sequences with long contexts only (one sequence of 32,768 keys: 39.6 us with 16 splits against 53.8 with 8;
        # two: 54.7 with 12 against 64.8; at 2,048 keys 11.8 against 11.1)
        wide = min(splits, max(8, wide_cluster_blocks // (ctx.n_tokens * nkv)), ops.attention_decode_fused_max_splits(d, ctx.device))
        splits = wide if ctx.max_context > long_context_keys else 8
    ops.attention_decode_fused(qkv, cache.keys, cache.values, out, q_norm_w, k_norm_w, cos, sin, eps, ctx.token_seq,
                               ctx.token_pos, table, ctx.n_tokens, nq, nkv, d, part.scale, part.window, splits,
                               write_kv=not cache.shared)
    return True


def _projection_pair_kernel(part, x, cache, q, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool:
    """The q/k/v product on pairs of SMs with norm, rotation and the cache write in its epilogue, where `linear`
    would take the persistent pairs kernel anyway: head sizes 64, 128 and 256, the whole head rotated."""
    from . import linear as linear_module
    nq, nkv, d = part.num_heads, part.num_kv_heads, part.head_dim
    N, K = ctx.n_tokens, part.hidden_size
    if d not in ops.PAIR_QKV_HEAD_DIMS or K % 8 != 0 or N < fused_projection_rows:
        return False
    if cos is not None and 2 * cos.shape[-1] != d:
        return False
    if linear_module.set_bf16_kernel_active() or linear_module.tcgen05_form(N, (nq + 2 * nkv) * d, K) != "pair" \
            or linear_module.pair_plan(N, (nq + 2 * nkv) * d, K)[1] != 1:
        return False
    ops.gemm_tcgen05_pair_qkv(x, part.w_qkv, q, cache.keys, cache.values, q_norm_w, k_norm_w, cos, sin, eps, ctx.token_seq,
                              ctx.token_pos, table, N, nq, nkv, d, write_kv=not cache.shared)
    return True


_sm_counts = {}


def _sm_count(device) -> int:
    device = torch.device(device)
    count = _sm_counts.get(device)
    if count is None:
        count = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return count


def _prefill_flash_kernel(part, q, cache, out, ctx, table) -> bool:
    """The tiled tensor-core kernel for steps that bring prompts (or any mix of lengths)."""
    ops.attention_prefill(q, cache.keys, cache.values, out, ctx.seq_start, ctx.seq_pos0, table, ctx.n_seqs,
                          ctx.max_new, part.num_heads, part.num_kv_heads, part.head_dim, part.scale, part.window)
    return True


def _prefill_tcgen05_kernel(part, q, cache, out, ctx, table) -> bool:
    """Both products of the attention on tcgen05 with TMA-fed tiles: head sizes 64 and 128, no window,
    and enough new tokens for 128-row tiles to be worth it."""
    if not ops.attention_prefill_tc_fits(part.head_dim, part.window) or ctx.max_new < tc_prefill_rows or part.scale <= 0:
        return False
    ops.attention_prefill_tc(q[:ctx.n_tokens], cache.keys, cache.values, out, ctx.seq_start, ctx.seq_pos0, table,
                             ctx.n_seqs, ctx.max_new, ctx.n_tokens, part.num_heads, part.num_kv_heads, part.head_dim,
                             part.scale)
    return True


long_context_keys = 4096  # a decode step whose sequences may be longer takes wider clusters (if they are few)
wide_cluster_blocks = 200 # blocks of a decode step with clusters beyond the portable size
tc_prefill_rows = 128     # from this many new tokens of the longest sequence on, the tcgen05 kernel runs
# From this many tokens in a step on, the q/k/v product does norm, rotation and cache write in its epilogue: with
# several tiles per pair of SMs the longer epilogue hides under the next tile's K steps (measured: 8,192 tokens
# 321-338 us against 381-412 for product + qkv_prepare, 2,048 tokens 83.5 against 86, 512 tokens 41 against 34).
fused_projection_rows = 2048

DECODE_KERNELS.append(_decode_split_kernel)
FUSED_DECODE_KERNELS.append(_decode_fused_kernel)
FUSED_PROJECTION_KERNELS.append(_projection_pair_kernel)
PREFILL_KERNELS.append(_prefill_tcgen05_kernel)
PREFILL_KERNELS.append(_prefill_flash_kernel)

register_part("mixer", "gqa_attention", GQAAttention)
