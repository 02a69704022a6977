"""Configuration: the reference's fixtures, required keys, strict types, rejected options,
the registry, and the plan as data."""
import copy
import json
import os

import pytest

import qwen3_b200 as q
from helpers import TINY, tiny

FIXTURES = os.path.join(os.path.dirname(__file__), "golden", "fixtures")


def test_reference_fixture_8b():
    # values asserted by the reference's tests/unit/model_config_test.cpp
    c = q.load_config(os.path.join(FIXTURES, "qwen3_8b.json"))
    assert (c.hidden_size, c.num_hidden_layers, c.q_projection_size, c.kv_projection_size) == (4096, 36, 4096, 1024)
    assert c.query_heads_per_kv_head == 4 and c.tie_word_embeddings is False
    assert c.vocab_size == 151936 and c.intermediate_size == 12288 and c.head_dim == 128
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-6 and c.max_position_embeddings == 40960


def test_from_json_reads_a_file_or_its_folder(tmp_path):
    path = os.path.join(FIXTURES, "qwen3_8b.json")
    assert q.Qwen3Config.from_json(path) == q.load_config(path)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(tiny("A"), f)
    assert q.Qwen3Config.from_json(str(tmp_path), strict=True) == q.config_from_dict(tiny("A"))
    with pytest.raises(q.ConfigError):
        q.Qwen3Config.from_json(str(tmp_path / "absent.json"))


def test_reference_fixture_0_6b_head_dim_is_not_hidden_over_heads():
    c = q.load_config(os.path.join(FIXTURES, "qwen3_0_6b.json"))
    assert (c.hidden_size, c.num_hidden_layers, c.q_projection_size, c.kv_projection_size) == (1024, 28, 2048, 1024)
    assert c.query_heads_per_kv_head == 2 and c.tie_word_embeddings is True


@pytest.mark.parametrize("layers,hidden,heads,inter,params_b", [(40, 5120, 40, 17408, 14.77), (64, 5120, 64, 25600, 32.76)])
def test_larger_shapes_of_the_family_parse_and_plan(layers, hidden, heads, inter, params_b):
    """The 14B and 32B shapes (same keys as the 8B fixture, other sizes): derived sizes, the plan's tensor
    list and its parameter count."""
    with open(os.path.join(FIXTURES, "qwen3_8b.json")) as f:
        root = json.load(f)
    root.update(num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads, intermediate_size=inter)
    c = q.config_from_dict(root, strict=True)
    assert (c.q_projection_size, c.kv_projection_size, c.query_heads_per_kv_head) == (heads * 128, 1024, heads // 8)
    specs = q.build_model(c.plan()).weight_specs()
    assert len(specs) == 2 + 11 * layers + 1                      # src/model/weights.cpp:83,123 (untied)
    count = sum(int(__import__("math").prod(s.shape)) for s in specs.values())
    assert abs(count / 1e9 - params_b) < 0.01


def test_golden_accept_reject_matches_the_reference_parser():
    """tests/golden/config_cases.json was produced by the reference's own src/model/config.cpp
    compiled on the CPU (tests/golden/make_config_golden.py); both parsers must agree on every case."""
    with open(os.path.join(os.path.dirname(__file__), "golden", "config_cases.json")) as f:
        cases = json.load(f)
    assert len(cases) >= 20
    for case in cases:
        try:
            c = q.config_from_dict(case["config"], strict=True)
            ok = True
        except q.ConfigError:
            ok = False
        assert ok == case["reference_accepts"], case["name"]
        if ok:
            ref = case["reference_values"]
            assert [c.num_hidden_layers, c.hidden_size, c.q_projection_size, c.kv_projection_size,
                    c.query_heads_per_kv_head, int(c.tie_word_embeddings)] == ref[:6], case["name"]


@pytest.mark.parametrize("name", list(TINY))
def test_round_trip_and_plan(name):
    c = q.config_from_dict(tiny(name))
    assert q.config_from_dict(c.to_dict()) == c
    plan = c.plan()
    assert plan.order == list(range(c.num_hidden_layers)) and len(plan.layers) == c.num_hidden_layers
    mixer = plan.layers[0].mixer
    assert mixer.kind == "gqa_attention" and mixer.params["head_dim"] == c.head_dim
    assert mixer.params["qk_norm"].params == {"size": c.head_dim, "eps": c.rms_norm_eps}
    assert mixer.params["position"].params["theta"] == c.rope_theta
    assert plan.layers[0].feed_forward.params["intermediate_size"] == c.intermediate_size
    assert plan.head.params["tied_to"] == ("model.embed_tokens.weight" if c.tie_word_embeddings else None)
    assert plan.stop_token_ids == [c.eos_token_id, c.bos_token_id]
    specs = q.build_model(plan).weight_specs()
    assert len(specs) == 2 + 11 * c.num_hidden_layers + (0 if c.tie_word_embeddings else 1)
    assert specs["model.layers.0.self_attn.q_proj.weight"].shape == (c.num_attention_heads * c.head_dim, c.hidden_size)
    assert specs["model.layers.0.self_attn.k_norm.weight"].shape == (c.head_dim,)


REQUIRED = ["model_type", "architectures", "hidden_act", "torch_dtype", "vocab_size", "hidden_size",
            "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
            "max_position_embeddings", "rope_theta", "rms_norm_eps", "bos_token_id", "eos_token_id",
            "attention_bias", "tie_word_embeddings", "use_sliding_window"]


@pytest.mark.parametrize("key", REQUIRED)
def test_every_key_is_required(key):
    cfg = tiny("A")
    del cfg[key]
    with pytest.raises(q.ConfigError, match=key):
        q.config_from_dict(cfg, strict=True)


def test_config_files_of_newer_exporters_are_read():
    """`dtype` for `torch_dtype`, `rope_parameters` for `rope_theta`, absent switches, a window size kept
    beside use_sliding_window = false: accepted by default, refused by the strict (reference) mode."""
    cfg = tiny("B")
    for key in ("torch_dtype", "rope_theta", "attention_bias", "use_sliding_window", "hidden_act", "bos_token_id",
                "tie_word_embeddings", "rope_scaling"):
        del cfg[key]
    cfg.update(dtype="bfloat16", rope_parameters={"rope_type": "default", "rope_theta": 1000000.0},
               sliding_window=4096, eos_token_id=[5, 7], layer_types=["full_attention"] * 3)
    c = q.config_from_dict(cfg)
    assert c == q.config_from_dict(tiny("B", bos_token_id=5))
    with pytest.raises(q.ConfigError):
        q.config_from_dict(cfg, strict=True)
    with pytest.raises(q.ConfigError):
        q.config_from_dict(dict(cfg, rope_parameters={"rope_type": "yarn", "rope_theta": 1e6, "factor": 4.0}))
    del cfg["head_dim"]
    assert q.config_from_dict(cfg).head_dim == 96 // 8
    for size in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                 "rms_norm_eps", "max_position_embeddings"):
        broken = dict(cfg)
        del broken[size]
        with pytest.raises(q.ConfigError, match=size):
            q.config_from_dict(broken)


@pytest.mark.parametrize("key,value", [
    ("vocab_size", 256.0), ("vocab_size", "256"), ("vocab_size", True), ("hidden_size", 2 ** 31),
    ("rope_theta", "1e6"), ("rope_theta", 1e39), ("rms_norm_eps", None), ("tie_word_embeddings", 1),
    ("attention_bias", "false"), ("model_type", 3), ("architectures", "Qwen3ForCausalLM"),
])
def test_strict_types(key, value):
    with pytest.raises(q.ConfigError):
        q.config_from_dict(tiny("A", **{key: value}))


@pytest.mark.parametrize("changes", [
    {"num_key_value_heads": 3}, {"head_dim": 15}, {"vocab_size": 0}, {"num_hidden_layers": -1},
    {"rope_theta": 0}, {"rms_norm_eps": 0.0}, {"bos_token_id": 384}, {"eos_token_id": -1},
    {"attention_bias": True}, {"use_sliding_window": True}, {"sliding_window": 4096},
    {"rope_scaling": {"type": "yarn", "factor": 4.0}}, {"quantization_config": {"bits": 4}},
    {"hidden_act": "gelu"}, {"torch_dtype": "float16"}, {"model_type": "qwen3_moe"},
    {"architectures": ["Qwen3MoeForCausalLM"]}, {"architectures": []},
])
def test_rejected_options(changes):
    with pytest.raises(q.ConfigError):
        q.config_from_dict(tiny("B", **changes), strict=True)
    if changes != {"sliding_window": 4096}:         # a window size beside use_sliding_window = false is unused
        with pytest.raises(q.ConfigError):
            q.config_from_dict(tiny("B", **changes))


def test_rope_theta_may_be_a_json_integer_and_null_options_are_fine():
    c = q.config_from_dict(tiny("B", rope_theta=1000000, quantization_config=None))
    assert c.rope_theta == 1e6 and isinstance(c.rope_theta, float)


def test_registry_unknown_architecture_lists_known_ones(tmp_path):
    with pytest.raises(q.ConfigError, match="Qwen3ForCausalLM"):
        q.config_from_dict(tiny("A", architectures=["LlamaForCausalLM"], model_type="llama"))
    with pytest.raises(q.ConfigError, match="cannot open"):
        q.load_config(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(q.ConfigError, match="parse"):
        q.load_config(str(tmp_path))


def test_a_new_architecture_registers_without_touching_the_library():
    class ToyConfig:
        @classmethod
        def from_dict(cls, root):
            c = cls()
            c.width = root["width"]
            return c

        def to_dict(self):
            return {"architectures": ["ToyForCausalLM"], "width": self.width}

        def plan(self):
            raise NotImplementedError

    q.register_architecture("ToyForCausalLM", ToyConfig)
    try:
        assert q.config_from_dict({"architectures": ["ToyForCausalLM"], "width": 7}).width == 7
        assert "ToyForCausalLM" in q.known_architectures()
    finally:
        from qwen3_b200.config import registry
        registry._ARCHITECTURES.pop("ToyForCausalLM")


def test_plan_checks_order_and_cache_sharing():
    c = q.config_from_dict(tiny("A"))
    plan = c.plan()
    import dataclasses
    with pytest.raises(ValueError):
        dataclasses.replace(plan, order=[0, 2])
    twice = dataclasses.replace(plan, order=[0, 1, 0])
    assert twice.order == [0, 1, 0]
    shared = dataclasses.replace(plan, layers=[plan.layers[0], dataclasses.replace(plan.layers[1], cache_from=0)])
    assert shared.layers[1].cache_from == 0
    with pytest.raises(ValueError):
        dataclasses.replace(plan, layers=[dataclasses.replace(plan.layers[0], cache_from=1), plan.layers[1]])


def test_a_head_size_the_kernels_do_not_take_is_refused_when_the_model_is_planned():
    """config.json may hold any even head size (the reference's own rule), so parsing accepts it; the plan,
    which is the first thing an engine asks for, says what this library runs."""
    import qwen3_b200 as q
    cfg = dict(tiny("A"), head_dim=24)
    config = q.config_from_dict(cfg)
    assert config.head_dim == 24
    with pytest.raises(q.ConfigError, match="multiples of 16"):
        config.plan()
    with pytest.raises(q.ConfigError, match="multiples of 16"):
        q.config_from_dict(dict(cfg, head_dim=272)).plan()
