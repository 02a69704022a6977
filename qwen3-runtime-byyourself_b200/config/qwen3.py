"""Typed configuration of the Qwen3 dense decoder, read from its config.json keys.

Parity with the reference (RicardoMin/Qwen3-Runtime-ByYourself):
  fields             include/qwen3/model/config.h:8-50
  required keys      src/model/config.cpp:252-343 (no model size has a default)
  strict JSON types  src/model/config.cpp:40-121
  validation         src/model/config.cpp:175-250
  rejected options   attention_bias, use_sliding_window (:239-249), non-null
                     rope_scaling / sliding_window / quantization_config (:299-301),
                     hidden_act other than silu (:285-289)
Beyond the reference: torch_dtype may be "float32" as well as "bfloat16" (a
folder of 32-bit weights for the 32-bit path), and `plan()` states the model as
data for the parts, the cache and the step function.

`from_dict(root, strict=True)` is the reference's parser key for key.  The default
(`strict=False`, what `load_config` uses) additionally reads config.json files as
newer exporters write them: `dtype` for `torch_dtype`, `rope_parameters.rope_theta`
for `rope_theta`, and it lets the switches that have one possible value here be absent
(`attention_bias`, `use_sliding_window`, `hidden_act`, `tie_word_embeddings` = false,
`bos_token_id`, `head_dim` = hidden_size / num_attention_heads).  Every model size and
`rms_norm_eps` stay required in both modes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict

from .plan import LayerSpec, ModelPlan, PartSpec
from .registry import ConfigError, register_architecture

_INT32_MIN, _INT32_MAX = -(2 ** 31), 2 ** 31 - 1
_FLOAT32_MAX = 3.4028234663852886e38


def _required(root, key):
    if key not in root:
        raise ConfigError(f"missing required config field '{key}'")
    return root[key]


def _int32(root, key):
    v = _required(root, key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config field '{key}' must be an integer")
    if not _INT32_MIN <= v <= _INT32_MAX:
        raise ConfigError(f"config field '{key}' is outside the int32 range")
    return v


def _float(root, key):
    v = _required(root, key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config field '{key}' must be numeric")
    v = float(v)
    if not math.isfinite(v) or abs(v) > _FLOAT32_MAX:
        raise ConfigError(f"config field '{key}' cannot be represented as float")
    return v


def _bool(root, key):
    v = _required(root, key)
    if not isinstance(v, bool):
        raise ConfigError(f"config field '{key}' must be boolean")
    return v


def _string(root, key):
    v = _required(root, key)
    if not isinstance(v, str):
        raise ConfigError(f"config field '{key}' must be a string")
    return v


def _reject_non_null(root, key):
    if root.get(key) is not None:
        raise ConfigError(f"config field '{key}' is not supported and must be null or absent")


def _with_defaults(root: dict) -> dict:
    """The same keys as the strict parser reads, filled from the spellings of newer exporters and from
    the only value this architecture allows where a switch is absent."""
    if not isinstance(root, dict):
        return root
    out = dict(root)
    if "torch_dtype" not in out:
        out["torch_dtype"] = out.get("dtype") if isinstance(out.get("dtype"), str) else "bfloat16"
    rope = out.get("rope_parameters")
    if isinstance(rope, dict):
        if rope.get("rope_type", rope.get("type", "default")) not in ("default", None):
            raise ConfigError("config field 'rope_parameters' asks for a rope scaling that is not supported")
        if "rope_theta" not in out and "rope_theta" in rope:
            out["rope_theta"] = rope["rope_theta"]
    if isinstance(out.get("rope_scaling"), dict) and out["rope_scaling"].get("rope_type", out["rope_scaling"].get("type")) in ("default", None):
        out["rope_scaling"] = None
    out.setdefault("hidden_act", "silu")
    out.setdefault("attention_bias", False)
    out.setdefault("use_sliding_window", False)
    out.setdefault("tie_word_embeddings", False)
    if not out.get("use_sliding_window"):
        out["sliding_window"] = None            # exporters keep the window size next to use_sliding_window = false
    if "head_dim" not in out and isinstance(out.get("hidden_size"), int) and isinstance(out.get("num_attention_heads"), int) \
            and out["num_attention_heads"] > 0:
        out["head_dim"] = out["hidden_size"] // out["num_attention_heads"]
    if "num_key_value_heads" not in out and "num_attention_heads" in out:
        out["num_key_value_heads"] = out["num_attention_heads"]
    if isinstance(out.get("eos_token_id"), list) and out["eos_token_id"]:
        out["eos_token_id"] = out["eos_token_id"][0]
    for key in ("bos_token_id", "eos_token_id"):
        if out.get(key) is None:
            out[key] = out.get("eos_token_id") if key == "bos_token_id" and isinstance(out.get("eos_token_id"), int) else 0
    return out


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    bos_token_id: int
    eos_token_id: int
    tie_word_embeddings: bool
    attention_bias: bool = False
    use_sliding_window: bool = False
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    # -- derived sizes (include/qwen3/model/config.h:36-46)
    @property
    def q_projection_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_projection_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def query_heads_per_kv_head(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # -- parsing
    @classmethod
    def from_dict(cls, root: dict, strict: bool = False) -> "Qwen3Config":
        if not strict:
            root = _with_defaults(root)
        if _string(root, "model_type") != cls.model_type:
            raise ConfigError("only Qwen3 dense models are supported (model_type must be 'qwen3')")
        if cls.architecture not in [a for a in _required(root, "architectures") if isinstance(a, str)]:
            raise ConfigError(f"only {cls.architecture} is supported")
        hidden_act = _string(root, "hidden_act")
        torch_dtype = _string(root, "torch_dtype")
        for key in ("rope_scaling", "sliding_window", "quantization_config"):
            _reject_non_null(root, key)
        config = cls(
            vocab_size=_int32(root, "vocab_size"),
            hidden_size=_int32(root, "hidden_size"),
            intermediate_size=_int32(root, "intermediate_size"),
            num_hidden_layers=_int32(root, "num_hidden_layers"),
            num_attention_heads=_int32(root, "num_attention_heads"),
            num_key_value_heads=_int32(root, "num_key_value_heads"),
            head_dim=_int32(root, "head_dim"),
            max_position_embeddings=_int32(root, "max_position_embeddings"),
            rope_theta=_float(root, "rope_theta"),
            rms_norm_eps=_float(root, "rms_norm_eps"),
            bos_token_id=_int32(root, "bos_token_id"),
            eos_token_id=_int32(root, "eos_token_id"),
            attention_bias=_bool(root, "attention_bias"),
            tie_word_embeddings=_bool(root, "tie_word_embeddings"),
            use_sliding_window=_bool(root, "use_sliding_window"),
            hidden_act=hidden_act,
            torch_dtype=torch_dtype,
        )
        config.validate()
        return config

    @classmethod
    def from_json(cls, path: str, strict: bool = False) -> "Qwen3Config":
        """Read a config.json (or the folder that holds it) as this architecture's configuration."""
        import json
        import os
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        try:
            with open(path, "r", encoding="utf-8") as f:
                root = json.load(f)
        except OSError as e:
            raise ConfigError(f"cannot open model config: {path}: {e}") from None
        except json.JSONDecodeError as e:
            raise ConfigError(f"cannot parse model config {path!r}: {e}") from None
        if not isinstance(root, dict):
            raise ConfigError("model config root must be a JSON object")
        return cls.from_dict(root, strict=strict)

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be positive")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2 != 0:
            raise ConfigError("head_dim must be even for RoPE")
        if not (math.isfinite(self.rope_theta) and self.rope_theta > 0):
            raise ConfigError("rope_theta must be finite and positive")
        if not (math.isfinite(self.rms_norm_eps) and self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be finite and positive")
        for key in ("bos_token_id", "eos_token_id"):
            if not 0 <= getattr(self, key) < self.vocab_size:
                raise ConfigError(f"{key} is outside the vocabulary")
        if self.attention_bias:
            raise ConfigError("attention bias is not supported")
        if self.use_sliding_window:
            raise ConfigError("sliding-window attention is not supported")
        if self.hidden_act != "silu":
            raise ConfigError("only the SiLU activation is supported")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError("only bfloat16 (or float32) Qwen3 checkpoints are supported")

    def to_dict(self) -> dict:
        """The keys of a config.json that `from_dict` reads back to an equal object."""
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = self.model_type
        d["rope_scaling"] = None
        d["sliding_window"] = None
        return d

    # -- the model as data
    def plan(self) -> ModelPlan:
        H, d, eps = self.hidden_size, self.head_dim, self.rms_norm_eps
        if d % 16 != 0 or d > 256:
            # config.json allows any even head size (src/model/config.cpp:205-209); this library's attention
            # kernels are tiled in steps of 16, so the model is refused here, before any weight is read
            raise ConfigError(f"head_dim {d}: this library runs head sizes that are multiples of 16, up to 256")
        norm = PartSpec("rms_norm", {"size": H, "eps": eps})
        mixer = PartSpec("gqa_attention", {
            "hidden_size": H,
            "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads,
            "head_dim": d,
            "scale": d ** -0.5,
            "qk_norm": PartSpec("rms_norm", {"size": d, "eps": eps}),
            "position": PartSpec("rope", {"head_dim": d, "theta": self.rope_theta,
                                          "max_positions": self.max_position_embeddings}),
            "window": None,
            "prefix": "self_attn.",
        })
        feed_forward = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": self.intermediate_size,
                                           "prefix": "mlp."})
        block = PartSpec("pre_norm", {"norm": norm,
                                      "mixer_norm_name": "input_layernorm.weight",
                                      "feed_forward_norm_name": "post_attention_layernorm.weight"})
        layers = [LayerSpec(block=block, mixer=mixer, feed_forward=feed_forward, prefix=f"model.layers.{i}.")
                  for i in range(self.num_hidden_layers)]
        return ModelPlan(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=H,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H}),
            embedding_prefix="model.embed_tokens.",
            layers=layers,
            order=list(range(self.num_hidden_layers)),
            final_norm=norm,
            final_norm_prefix="model.norm.",
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": H,
                                      "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None}),
            head_prefix="lm_head.",
            stop_token_ids=[self.eos_token_id, self.bos_token_id],
        )


register_architecture(Qwen3Config.architecture, Qwen3Config)
