"""A model put together from a `ModelPlan`: embedding, layers in their order, final norm, head.

The forward pass is the reference's (src/model/model.cpp:107-147: embedding ->
layers -> final norm) followed by the output projection (src/model/lm_head.cpp:
188-191), with two differences of arrangement: it runs on packed tokens of several
sequences of unequal length, and the final norm and the head run only on the rows
whose logits are wanted (the reference normalises every row and drops all but the
last).
"""
from __future__ import annotations

import sys
from typing import Dict, List, Optional

import torch

from ..cache.book import CacheNeed
from ..config.plan import ModelPlan
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import build_part


class Model:
    def __init__(self, plan: ModelPlan):
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding)
        self.blocks = []
        for spec in plan.layers:
            mixer = build_part("mixer", spec.mixer)
            feed_forward = build_part("feed_forward", spec.feed_forward)
            self.blocks.append(build_part("block", spec.block, mixer, feed_forward))
        self.final_norm = build_part("norm", plan.final_norm)
        self.head = build_part("head", plan.head)
        self.dtype: Optional[torch.dtype] = None
        self.device = None
        self._warned_rounding = False

    # -- weights
    def weight_specs(self) -> Dict[str, WeightSpec]:
        p = self.plan
        specs = dict(self.embedding.weight_specs(p.embedding_prefix))
        for spec, block in zip(p.layers, self.blocks):
            specs.update(block.weight_specs(spec.prefix))
        specs.update(self.final_norm.weight_specs(p.final_norm_prefix + "weight"))
        specs.update(self.head.weight_specs(p.head_prefix))
        return specs

    def ignorable_names(self) -> List[str]:
        return list(getattr(self.head, "ignorable", lambda prefix: [])(self.plan.head_prefix))

    def bind(self, weights, dtype: torch.dtype, device) -> None:
        """Take the tensors (by checkpoint name) for computing in `dtype` on `device`.  `weights` is a dict of
        tensors, or a checkpoint that uploads on demand (`weights.loader.open_upload`).

        Matrices are used in the compute type: a bfloat16 checkpoint widens exactly for
        the 32-bit path; a 32-bit matrix is rounded to bfloat16 for a bfloat16 engine, with
        one line on stderr saying so.  Scale vectors are always read as float32."""
        from ..weights.upload import TensorDict
        if isinstance(weights, dict):
            weights = TensorDict(weights, self.weight_specs(), dtype, device, self._warn_rounding)
        p = self.plan
        self.dtype, self.device = dtype, torch.device(device)
        self.embedding.bind(weights, p.embedding_prefix, dtype, device)
        self.final_norm.bind(weights, p.final_norm_prefix + "weight", dtype, device)
        self.head.bind(weights, p.head_prefix, dtype, device)
        for spec, block in zip(p.layers, self.blocks):
            block.bind(weights, spec.prefix, dtype, device)

    def _warn_rounding(self, name: str) -> None:
        if not self._warned_rounding:
            self._warned_rounding = True
            print(f"[qwen3_b200] {name} (and other matrices) are stored in 32-bit and are rounded to bfloat16 "
                  f"for the bfloat16 kernels; use dtype float32 to compute with them as stored", file=sys.stderr)

    # -- cache
    def cache_needs(self) -> List[Optional[CacheNeed]]:
        return [None if spec.cache_from is not None else block.mixer.cache_need()
                for spec, block in zip(self.plan.layers, self.blocks)]

    def cache_sources(self) -> Dict[int, int]:
        return {i: spec.cache_from for i, spec in enumerate(self.plan.layers) if spec.cache_from is not None}

    # -- one step over packed tokens
    def forward(self, ctx, cache) -> Optional[torch.Tensor]:
        """Runs the step's tokens through every layer (filling the cache); returns float32
        logits [n_want, vocab] for the wanted rows, or None if none is wanted."""
        N, H = ctx.n_tokens, self.plan.hidden_size
        residual = ctx.scratch.get("model.residual", (N, H), ctx.dtype)
        self.embedding.forward(ctx.token_ids[:N], residual)
        delta = None
        for index in self.plan.order:
            residual, delta = self.blocks[index].forward(residual, delta, ctx, cache.layer(index))
        if ctx.n_want == 0:
            return None
        R = ctx.n_want
        normed = ctx.scratch.get("model.rows_normed", (R, H), ctx.dtype)
        if ctx.want_all:                                   # a decode step: the last residual sum rides in the norm
            self.final_norm(residual, normed, delta)
        else:
            rows = ctx.scratch.get("model.rows", (R, H), ctx.dtype)
            ops.gather_rows(residual, ctx.want_rows[:R], rows, delta)
            self.final_norm(rows, normed)
        logits = ctx.scratch.get("model.logits", (R, self.plan.vocab_size), torch.float32)
        return self.head.forward(normed, logits)


def build_model(plan: ModelPlan) -> Model:
    return Model(plan)
