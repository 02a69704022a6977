"""Parts of a model (norm, position encoding, mixer, feed-forward, block, embedding, head)
and the model that a plan puts together from them."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Part, build_part,
                   register_part)
from . import norm, position, attention, mlp, block, embedding  # noqa: F401  (registration)
from .model import Model, build_model

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Part", "build_part",
           "register_part", "Model", "build_model"]
