"""Token embedding and output head as parts.

Embedding: a row gather (src/ops/embedding.cu:38-52).  Head: logits = x . W^T with W
either `lm_head.weight` or, for tied checkpoints, the embedding table, in which case
`lm_head.weight` is not read (src/model/weights.cpp:116-118,198-204).  The reference
rounds logits to bfloat16 (src/ops/linear.cpp:118); here they leave the product as
float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import linear


class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.table = None

    def weight_specs(self, prefix: str) -> dict:
        return {prefix + "weight": WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        self.table = weights[prefix + "weight"].contiguous()

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        return ops.embedding(token_ids, self.table, out)


class LMHead(Part):
    def __init__(self, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None):
        self.vocab_size, self.hidden_size, self.tied_to = int(vocab_size), int(hidden_size), tied_to
        self.weight = None

    def weight_specs(self, prefix: str) -> dict:
        return {} if self.tied_to else {prefix + "weight": WeightSpec((self.vocab_size, self.hidden_size))}

    def ignorable(self, prefix: str):
        return [prefix + "weight"] if self.tied_to else []

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        self.weight = weights[self.tied_to if self.tied_to else prefix + "weight"].contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, out)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
