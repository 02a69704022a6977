"""bin/trace_run as a user runs it: a subprocess fed steps on standard input, logits read back
from <step>.f32 files, for the three cuttings, in 32-bit and in bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import schedules
from helpers import FP32_TOL, bf16_tolerance, make_folder, plain_logits, random_tokens, tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(folder, dtype, steps, rows, out_dir, vocab):
    max_tokens = schedules.peak_tokens(steps)
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                             "--out", out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    got = {}
    try:
        for step, out in zip(steps, rows):
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()          # the next step may come only after this line
            assert line == f"done {step['step']}", (line, proc.stderr.read()[-2000:] if proc.poll() is not None else "")
            path = os.path.join(out_dir, f"{step['step']}.f32")
            if out:
                block = np.fromfile(path, dtype="<f4").reshape(len(out), vocab)
                for key, row in zip(out, block):
                    got[key] = row
            else:
                assert not os.path.exists(path)
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0, proc.stderr.read()[-2000:]
    finally:
        if proc.poll() is None:
            proc.kill()
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_three_cuttings(tmp_path, dtype):
    cfg = tiny("B")
    folder, weights = make_folder(tmp_path, cfg, seed=41)
    rng = np.random.default_rng(7)
    lengths = [70, 33, 1, 130, 64]
    requests = {f"q{i}": random_tokens(rng, n, cfg["vocab_size"]) for i, n in enumerate(lengths)}
    prompts = dict(zip(requests, [10, 33, 1, 65, 63]))
    w_steps, w_rows = schedules.whole(requests)
    t_steps, t_rows = schedules.tail_one_by_one(requests, 32)
    b_steps, b_rows = schedules.batched(requests, prompts, 2)
    # one process replays all three one after the other: the cache is sized for the largest moment
    steps, rows = [], []
    for part_steps, part_rows in ((w_steps, w_rows), (t_steps, t_rows), (b_steps, b_rows)):
        for s, r in zip(part_steps, part_rows):
            steps.append(dict(s, step=len(steps)))
            rows.append([(f"{len(steps)}:{rid}", rid, p) for rid, p in r])
    flat_rows = [[(tag, p) for tag, _, p in r] for r in rows]
    got = replay(folder, dtype, steps, flat_rows, str(tmp_path / "out"), cfg["vocab_size"])
    exact = {rid: plain_logits(cfg, weights, toks) for rid, toks in requests.items()}
    tol = {rid: FP32_TOL if dtype == "float32" else bf16_tolerance(cfg, weights, toks, exact[rid])
           for rid, toks in requests.items()}
    checked = 0
    for r in rows:
        for tag, rid, p in r:
            err = float(np.max(np.abs(got[(tag, p)] - exact[rid][p])))
            assert err <= tol[rid], f"{dtype}: step-tag {tag} position {p}: {err:.3e} > {tol[rid]:.3e}"
            checked += 1
    assert checked == sum(lengths) + sum(min(n, 33) for n in lengths) + sum(n - prompts[r] + 1 for r, n in zip(requests, lengths))


def test_trace_run_refuses_a_broken_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny("A")))
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path), "--dtype",
                          "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"], input="", capture_output=True,
                         text=True, timeout=300)
    assert out.returncode != 0 and "model.safetensors" in out.stderr
