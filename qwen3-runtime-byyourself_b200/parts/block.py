"""The arrangement of a layer: pre-norm residual block.

x += mixer(norm(x)); x += feed_forward(norm(x))  (src/model/decoder_layer.cpp:63-98).
The hidden state travels as (residual, delta): each sum is done by the next norm's
kernel, which writes the new residual and its normalised copy in one pass.
"""
from __future__ import annotations

from ..config.plan import PartSpec
from .base import Part, build_part, register_part


class PreNormBlock(Part):
    def __init__(self, mixer, feed_forward, norm: PartSpec, mixer_norm_name: str, feed_forward_norm_name: str):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm = build_part("norm", norm)
        self.feed_forward_norm = build_part("norm", norm)
        self.mixer_norm_name, self.feed_forward_norm_name = mixer_norm_name, feed_forward_norm_name

    def weight_specs(self, prefix: str) -> dict:
        specs = {}
        specs.update(self.mixer_norm.weight_specs(prefix + self.mixer_norm_name))
        specs.update(self.feed_forward_norm.weight_specs(prefix + self.feed_forward_norm_name))
        specs.update(self.mixer.weight_specs(prefix))
        specs.update(self.feed_forward.weight_specs(prefix))
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        self.mixer_norm.bind(weights, prefix + self.mixer_norm_name, dtype, device)
        self.feed_forward_norm.bind(weights, prefix + self.feed_forward_norm_name, dtype, device)
        self.mixer.bind(weights, prefix, dtype, device)
        self.feed_forward.bind(weights, prefix, dtype, device)

    def forward(self, residual, delta, ctx, cache):
        normed = ctx.scratch.get("block.normed", residual.shape, ctx.dtype)
        self.mixer_norm(residual, normed, delta)
        mixed = self.mixer.forward(normed, ctx, cache)
        self.feed_forward_norm(residual, normed, mixed)
        return residual, self.feed_forward.forward(normed, ctx)


register_part("block", "pre_norm", PreNormBlock)
