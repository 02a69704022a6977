"""Shared by the tests: the tiny configurations, model folders in temporary places, and
the comparison of engine logits with the plain implementation."""
import copy
import json
import os

import numpy as np

from plain import qwen3_plain as plain

# Two tiny configurations that differ in every size and option, and a third with a head
# size and a vocabulary that are no power of two and room for long sequences.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "torch_dtype": "bfloat16",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "attention_bias": False,
    "use_sliding_window": False, "sliding_window": None, "rope_scaling": None, "bos_token_id": 1, "eos_token_id": 2,
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "torch_dtype": "bfloat16",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 160, "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "attention_bias": False,
    "use_sliding_window": False, "sliding_window": None, "rope_scaling": None, "bos_token_id": 3, "eos_token_id": 5,
}
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "torch_dtype": "bfloat16",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
    "intermediate_size": 112, "vocab_size": 301, "rope_theta": 500000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 1024, "attention_bias": False,
    "use_sliding_window": False, "sliding_window": None, "rope_scaling": None, "bos_token_id": 0, "eos_token_id": 300,
}
# Sizes that rule out every vector path: a width that is no multiple of 8, an intermediate size that
# is no multiple of 8 (no interleaved gate/up), an odd vocabulary; head size 64 (the tcgen05 attention).
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "torch_dtype": "bfloat16",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "intermediate_size": 60, "vocab_size": 333, "rope_theta": 20000.0, "rms_norm_eps": 2e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "attention_bias": False,
    "use_sliding_window": False, "sliding_window": None, "rope_scaling": None, "bos_token_id": 4, "eos_token_id": 9,
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


def tiny(name, **changes):
    cfg = copy.deepcopy(TINY[name])
    cfg.update(changes)
    return cfg


def make_folder(tmp_path, cfg, seed, name="model", storage="bfloat16"):
    """Write a random model folder through the library's random-weights mode; returns
    (folder, weights as float64 NumPy arrays by name)."""
    import torch
    import qwen3_b200 as q
    cfg = dict(cfg, torch_dtype=storage)
    config = q.config_from_dict(cfg)
    folder = os.path.join(str(tmp_path), name)
    tensors = q.write_random_model(folder, config, seed)
    weights = {k: v.to(torch.float64).numpy() for k, v in tensors.items()}
    return folder, weights


def random_tokens(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def plain_logits(cfg, weights, tokens, rnd=plain.identity):
    return plain.forward(cfg, weights, tokens, rnd=rnd, rnd_logits=plain.identity if rnd is not plain.identity else None)


def bf16_tolerance(cfg, weights, tokens, exact):
    """How far bfloat16 rounding at the reference's rounding points moves the logits of this
    very case, times a margin: the yardstick for the bfloat16 engine."""
    emulated = plain_logits(cfg, weights, tokens, rnd=plain.round_bf16)
    return 4.0 * float(np.max(np.abs(emulated - exact))) + 1e-6


FP32_TOL = 1e-4
