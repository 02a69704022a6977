"""Sampling options, with the reference's names, defaults and checks.

include/qwen3/generation/sampler.h:16-33 (SamplingConfig: mode, temperature 0.6,
top_k 20, top_p 0.95, seed 42, valid_vocab_size 0 = all) and the validation of
src/generation/sampler.cpp:57-95.
"""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    mode: str = "sample"            # "sample" or "greedy"
    temperature: float = 0.6        # score = logit / temperature; finite and > 0
    top_k: int = 20                 # 0 disables; every candidate that reaches the k-th best score stays
    top_p: float = 0.95             # in (0, 1]; 1 disables
    seed: int = 42
    valid_vocab_size: int = 0       # only ids below it can be chosen; 0 = the whole vocabulary

    def __post_init__(self):
        if self.mode not in ("sample", "greedy"):
            raise ValueError("unknown sampling mode")
        if self.valid_vocab_size < 0:
            raise ValueError("valid_vocab_size cannot be negative")
        if self.mode == "greedy":
            return
        if not (math.isfinite(self.temperature) and self.temperature > 0):
            raise ValueError("sampling temperature must be finite and positive")
        if self.top_k < 0:
            raise ValueError("sampling top_k cannot be negative")
        if not (math.isfinite(self.top_p) and 0 < self.top_p <= 1):
            raise ValueError("sampling top_p must be in the interval (0, 1]")

    @classmethod
    def greedy(cls, valid_vocab_size: int = 0) -> "SamplingParams":
        return cls(mode="greedy", valid_vocab_size=valid_vocab_size)


_M64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_for(seed: int, sequence_id: int, step: int) -> float:
    """The uniform number in [0, 1) that the sampling kernel draws for (seed, sequence, step):
    53 high bits of a hash, scaled by 2^-53 as in src/generation/sampler.cpp:45-54."""
    h = _splitmix64((_splitmix64((seed & _M64) ^ _splitmix64(sequence_id & _M64)) + (step & _M64)) & _M64)
    return (h >> 11) * (1.0 / 9007199254740992.0)
