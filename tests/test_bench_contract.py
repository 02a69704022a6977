"""What bench.py owes its caller without a GPU: more than one GPU is refused with one line and exit code 2, the
reference arm says in one JSON line why it is unavailable, the shapes are those BASELINE.json names, and the byte and
flop counts behind the roofline figures are the sums they claim to be."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line():
    for n in ("2", "8"):
        out = run("--gpus", n, "--steps", "2", "--warmup", "1")
        assert out.returncode == 2
        assert len(out.stdout.strip().splitlines()) == 1 and "one GPU" in out.stdout


def test_the_reference_arm_says_why_it_is_unavailable():
    out = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert out.returncode == 0
    line = json.loads(out.stdout.strip())
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_shapes_and_counts():
    import bench
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        baseline = json.load(f)
    import re
    named = baseline["configs"][2]                          # a sentence that names every size
    cfg, context, batch = bench.SHAPES["8b"]
    for pattern, key in ((r"(\d+) layers", "num_hidden_layers"), (r"hidden (\d+)", "hidden_size"), (r"(\d+) q heads", "num_attention_heads"),
                         (r"(\d+) kv heads", "num_key_value_heads"), (r"head_dim (\d+)", "head_dim"),
                         (r"intermediate (\d+)", "intermediate_size"), (r"vocab (\d+)", "vocab_size")):
        found = re.search(pattern, named)
        assert found is not None and cfg[key] == int(found.group(1)), key
    assert context == int(re.search(r"context length is ([\d,]+)", named).group(1).replace(",", ""))
    assert batch == 8
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d, L = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    per_layer = (nq + 2 * nkv) * d * H + H * nq * d + 3 * H * I
    # every weight once in bfloat16, the norms' scale vectors in float32, the embedding rows of the step's tokens
    want = L * (per_layer * 2 + (2 * H + 2 * d) * 4) + V * H * 2 + H * 4 + 8 * H * 2
    assert bench.weight_bytes_per_step(cfg, L, 8) == want
    T = 2048
    flops = L * (2 * T * per_layer + 4 * nq * d * (T * (T + 1) // 2)) + 2 * V * H
    assert bench.prefill_flops(cfg, L, T) == flops
    peaks = bench.load_peaks()
    assert peaks["hbm_gbs"] > 1000 and peaks["bf16_tflops"] > 100
