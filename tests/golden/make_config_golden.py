"""Makes tests/golden/config_cases.json with the reference's own configuration parser.

Only this part of RicardoMin/Qwen3-Runtime-ByYourself compiles on a CPU-only machine (its model
code needs the absent `qwen3/core` headers, CUDA and cuBLAS), so it is the one place where the
library is compared with reference code rather than with reference formulas.

    python tests/golden/make_config_golden.py /path/to/reference

Compiles <reference>/src/model/config.cpp with config_probe.cpp, runs it on a list of
configurations (the tiny test models, the reference's fixtures, and one variation per rule) and
records for each whether the reference accepts it and the sizes it derives.
"""
import copy
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from helpers import TINY  # noqa: E402


def cases():
    out = []
    for name, cfg in TINY.items():
        out.append((f"tiny_{name}", copy.deepcopy(cfg)))
    for fixture in ("qwen3_0_6b.json", "qwen3_8b.json"):
        with open(os.path.join(HERE, "fixtures", fixture)) as f:
            out.append((fixture, json.load(f)))
    base = TINY["B"]
    variations = {
        "kv_heads_do_not_divide": {"num_key_value_heads": 3},
        "odd_head_dim": {"head_dim": 15},
        "zero_vocab": {"vocab_size": 0},
        "negative_layers": {"num_hidden_layers": -1},
        "zero_theta": {"rope_theta": 0},
        "zero_eps": {"rms_norm_eps": 0.0},
        "bos_outside": {"bos_token_id": 384},
        "eos_negative": {"eos_token_id": -1},
        "attention_bias": {"attention_bias": True},
        "use_sliding_window": {"use_sliding_window": True},
        "sliding_window_value": {"sliding_window": 4096},
        "rope_scaling": {"rope_scaling": {"type": "yarn", "factor": 4.0}},
        "quantization_config": {"quantization_config": {"bits": 4}},
        "quantization_config_null": {"quantization_config": None},
        "gelu": {"hidden_act": "gelu"},
        "float16": {"torch_dtype": "float16"},
        "moe_model_type": {"model_type": "qwen3_moe"},
        "other_architecture": {"architectures": ["Qwen3MoeForCausalLM"]},
        "no_architecture": {"architectures": []},
        "vocab_as_float": {"vocab_size": 384.0},
        "vocab_as_string": {"vocab_size": "384"},
        "theta_as_integer": {"rope_theta": 1000000},
        "theta_as_string": {"rope_theta": "1e6"},
        "tie_as_integer": {"tie_word_embeddings": 1},
        "hidden_too_large": {"hidden_size": 2 ** 31},
        "theta_beyond_float": {"rope_theta": 1e39},
    }
    for name, change in variations.items():
        cfg = copy.deepcopy(base)
        cfg.update(change)
        out.append((name, cfg))
    for key in ("head_dim", "rms_norm_eps", "tie_word_embeddings", "architectures", "torch_dtype"):
        cfg = copy.deepcopy(base)
        del cfg[key]
        out.append((f"missing_{key}", cfg))
    return out


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_config_golden.py REFERENCE_CHECKOUT")
    ref = sys.argv[1]
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "config_probe")
        subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ref, "include"),
                        "-I", os.path.join(ref, "third_party"), os.path.join(HERE, "config_probe.cpp"),
                        os.path.join(ref, "src", "model", "config.cpp"), "-o", exe], check=True)
        records = []
        for name, cfg in cases():
            path = os.path.join(tmp, "config.json")
            with open(path, "w") as f:
                json.dump(cfg, f)
            line = subprocess.run([exe, path], check=True, capture_output=True, text=True).stdout.strip()
            ok = line.startswith("OK ")
            rec = {"name": name, "config": cfg, "reference_accepts": ok, "reference_says": line}
            if ok:
                parts = line.split()[1:]
                rec["reference_values"] = [int(x) for x in parts[:6]] + [float(x) for x in parts[6:]]
            records.append(rec)
    with open(os.path.join(HERE, "config_cases.json"), "w") as f:
        json.dump(records, f, indent=1)
    print(f"{len(records)} cases, {sum(r['reference_accepts'] for r in records)} accepted by the reference")


if __name__ == "__main__":
    main()
