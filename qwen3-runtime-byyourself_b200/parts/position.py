"""Rotary position encoding as a part.

Table as in the reference (src/ops/rope.cu:276-295): inv_freq_i = theta^(-2i/d),
angle = position * inv_freq_i computed in float64, cosine and sine stored as
float32.  Rotation is half-split, pairs (i, i + d/2) (src/ops/rope.cu:60-84); the
attention part hands the tables to its fused kernel, `apply_` is the stand-alone form.
"""
from __future__ import annotations

import math

import torch

from .base import Part, register_part


class RotaryEmbedding(Part):
    fused_tables = True   # exposes cos/sin [positions, rotary_dim/2] float32 for a kernel to read

    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: int = 0):
        """`rotary_dim` (default: the head size, as in Qwen3): only the first `rotary_dim` values of a head are
        rotated, in pairs (i, i + rotary_dim/2) with inv_freq_i = theta^(-2i/rotary_dim); the rest pass through."""
        rotary_dim = int(rotary_dim) or int(head_dim)
        if head_dim % 2 or rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError("rotary encoding needs an even head_dim and an even rotary_dim within it")
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)
        self.rotary_dim = rotary_dim
        self.cos = self.sin = None

    def prepare(self, n_positions: int, device) -> None:
        n = min(int(n_positions), self.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n and self.cos.device == torch.device(device):
            return
        half = self.rotary_dim // 2
        # theta is held as a 32-bit float by the reference (include/qwen3/model/config.h:22)
        theta = float(torch.tensor(self.theta, dtype=torch.float32).item())
        inv_freq = torch.tensor([math.pow(theta, -(2.0 * i) / self.rotary_dim) for i in range(half)],
                                dtype=torch.float64)
        angle = torch.arange(n, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = torch.cos(angle).to(torch.float32).to(device).contiguous()
        self.sin = torch.sin(angle).to(torch.float32).to(device).contiguous()

    def apply_(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Rotate q [N, heads, d] and k in place (32-bit arithmetic, result in the tensors' type)."""
        half = self.rotary_dim // 2
        c = self.cos[positions.long()][:, None, :]
        s = self.sin[positions.long()][:, None, :]
        for t in (q, k):
            a, b = t[..., :half].float(), t[..., half:2 * half].float()
            first, second = a * c - b * s, b * c + a * s     # both from the unrotated values
            t[..., :half] = first.to(t.dtype)
            t[..., half:2 * half] = second.to(t.dtype)


register_part("position", "rope", RotaryEmbedding)
