"""SwiGLU feed-forward as a part: down( silu(gate(x)) * up(x) ).

Reference: src/model/mlp.cpp:101-115 (three products and one elementwise kernel) and
src/ops/elementwise.cu:47-65.  Here gate and up run as one product over one matrix made
at bind time, their rows interleaved in blocks of eight; for the few rows of a decode
step the product's kernel applies SiLU and the gating itself.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from ..weights.upload import fuse_interleaved, fuse_rows
from .base import Part, register_part
from . import linear as linear_module
from .linear import linear


class SwiGLU(Part):
    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = ""):
        self.hidden_size, self.intermediate_size, self.prefix = int(hidden_size), int(intermediate_size), prefix
        self.w_gate_up = self.w_down = None

    def weight_specs(self, prefix: str) -> dict:
        p, H, I = prefix + self.prefix, self.hidden_size, self.intermediate_size
        return {p + "gate_proj.weight": WeightSpec((I, H)), p + "up_proj.weight": WeightSpec((I, H)),
                p + "down_proj.weight": WeightSpec((H, I))}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p = prefix + self.prefix
        gate, up = p + "gate_proj.weight", p + "up_proj.weight"
        # gate and up rows interleaved in blocks of eight: one product gives both, and a kernel that owns
        # 16 consecutive output rows can finish silu(g) * u itself
        self.interleaved = self.intermediate_size % 8 == 0
        self.w_gate_up = fuse_interleaved(weights, gate, up, 8) if self.interleaved else fuse_rows(weights, [gate, up])
        self.w_down = weights.pop(p + "down_proj.weight").contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        N, I = ctx.n_tokens, self.intermediate_size
        act = ctx.scratch.get("ff.act", (N, I), ctx.dtype)
        fused = self.interleaved and ctx.dtype == torch.bfloat16 and self.hidden_size % 8 == 0
        if fused and N <= linear_module.skinny_rows:
            ops.gemm_skinny_gated(x, self.w_gate_up, act)          # product, SiLU and gating in one kernel
        elif fused and linear_module.tcgen05_form(N, 2 * I, self.hidden_size, gated=True) == "weights_first":
            ops.gemm_tcgen05_mid_gated(x, self.w_gate_up, act)     # gating where the cluster's partial tiles meet
        elif fused:
            ops.gemm_tcgen05_pair(x, self.w_gate_up, act, gated=True,  # the gating runs in the product's epilogue
                                  splits=linear_module.pair_plan(N, 2 * I, self.hidden_size)[1])
        else:
            gate_up = ctx.scratch.get("ff.gate_up", (N, 2 * I), ctx.dtype)
            linear(x, self.w_gate_up, gate_up)
            ops.silu_mul(gate_up, act, self.interleaved)
        out = ctx.scratch.get("ff.out", (N, self.hidden_size), ctx.dtype)
        return linear(act, self.w_down, out)


register_part("feed_forward", "swiglu", SwiGLU)
