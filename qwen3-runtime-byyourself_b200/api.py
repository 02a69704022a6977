"""The Python entry point.

    import qwen3_b200 as q
    engine = q.Engine.from_folder(model_dir, dtype="bfloat16", max_tokens=8 * 4096)
    results = q.generate_token_ids(engine, prompts, q.SamplingParams(mode="greedy"),
                                   q.GenerationOptions(max_new_tokens=64, stop_token_ids=[eos]))

Names follow the reference where it has them: `generate_token_ids`, `GenerationOptions`
(max_new_tokens 128, stop_token_ids), `GenerationResult` (token_ids, stop_reason)
(include/qwen3/generation/generator.h:15-46) and the sampling options of
include/qwen3/generation/sampler.h:16-33.  Unlike the reference, prompts are a list of
token-id lists of unequal length and are generated in batches.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from .cache import PAGE_TOKENS, CacheError, CacheFull, CacheNeed
from .config import (ConfigError, LayerSpec, ModelPlan, PartSpec, Qwen3Config, config_from_dict, known_architectures,
                     load_config, register_architecture)
from .engine.engine import Engine, StepEntry, StepError
from .engine.generate import MAX_NEW_TOKENS, STOP_TOKEN, GenerationResult, generate, plan_batches
from .parts import build_model, register_part
from .sampling import SamplingParams, uniform_for
from .weights import (SafetensorsFormatError, WeightError, WeightSpec, load_weights, random_weights, save_file,
                      write_model_folder, write_random_model)


@dataclass
class GenerationOptions:
    max_new_tokens: int = 128
    stop_token_ids: Sequence[int] = field(default_factory=list)


def generate_token_ids(engine: Engine, prompts: Sequence[Sequence[int]], sampling: Optional[SamplingParams] = None,
                       options: Optional[GenerationOptions] = None, batch_size: Optional[int] = None,
                       on_token=None, sequence_ids: Optional[Sequence[int]] = None) -> List[GenerationResult]:
    """Generate for every prompt (token ids in, new token ids out) on `engine`.  `sequence_ids` names the
    requests to the sampler (default: their index); a request draws the same tokens under the same name
    whatever else is in the batch."""
    from .sampling.sampler import Sampler
    sampling = sampling or SamplingParams()
    options = options or GenerationOptions()
    sampler = Sampler(sampling, engine.vocab_size, engine.device)
    return generate(engine, prompts, sampler, options.max_new_tokens, options.stop_token_ids, batch_size, on_token,
                    sequence_ids)


__all__ = [
    "PAGE_TOKENS", "CacheError", "CacheFull", "CacheNeed", "ConfigError", "LayerSpec", "ModelPlan", "PartSpec",
    "Qwen3Config", "config_from_dict", "known_architectures", "load_config", "register_architecture", "Engine",
    "StepEntry", "StepError", "MAX_NEW_TOKENS", "STOP_TOKEN", "GenerationResult", "generate", "plan_batches",
    "build_model", "register_part", "SamplingParams", "uniform_for", "SafetensorsFormatError", "WeightError",
    "WeightSpec", "load_weights", "random_weights", "save_file", "write_model_folder", "write_random_model",
    "GenerationOptions", "generate_token_ids",
]
