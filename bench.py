"""Benchmark of the library's headline metric: decoded tokens a second of a Qwen3-8B-shaped
model with random weights in bfloat16 on one B200, batch 8 at a context of 4,096 tokens.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 8b|14b|32b]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.
  value     decoded tokens a second, timed on the device with CUDA events around K steps;
            each step's next tokens are chosen on the device (greedy) and fed back there
  e2e       the same through the Python entry point `generate_token_ids`: host token ids in,
            host token ids out, every step
  prefill   one prompt of 2,048 tokens in one step: tokens a second, and its flops over the
            time over the bfloat16 peak
  roofline  bytes a decode step has to read (every weight it uses once, and the cache of the
            live requests) over its time, against the measured copy bandwidth
  points    decoded tokens a second at batch 1 and batch 64 (unequal prompts up to 2,048)
`--shape 14b` and `--shape 32b` run the same measurement on the two larger shapes of the baseline's
list (context 8,192 at batch 16; context 16,384 at batch 8), without the batch-1/64 points.
Peaks are read from MEASURED_PEAKS.json beside this file if it exists, else the stated
fallback of an earlier measurement on the same pool is used.
"""
import argparse
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "torch_dtype": "bfloat16",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 40960,
    "attention_bias": False, "use_sliding_window": False, "sliding_window": None, "rope_scaling": None,
    "bos_token_id": 151643, "eos_token_id": 151645,
}
# the further shapes of the baseline's list: (layers, hidden, q heads, intermediate), context, batch
SHAPES = {
    "8b": (dict(QWEN3_8B), 4096, 8),
    "14b": (dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408), 8192, 16),
    "32b": (dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600), 16384, 8),
}
PREFILL_TOKENS = 2048


def _number_under(raw, key):
    """The number stored under `key` in a JSON object, at the top or nested; a value that is itself an
    object is read through its 'value', 'median' or 'mean'."""
    if isinstance(raw, dict):
        if key in raw:
            v = raw[key]
            if isinstance(v, dict):
                for inner in ("value", "median", "mean"):
                    if isinstance(v.get(inner), (int, float)):
                        return float(v[inner])
            elif isinstance(v, (int, float)) and not isinstance(v, bool):
                return float(v)
        for v in raw.values():
            found = _number_under(v, key)
            if found is not None:
                return found
    return None


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS)
    hbm, flops = _number_under(raw, "hbm_gbs"), _number_under(raw, "bf16_tflops")
    if not hbm or not flops:
        return dict(FALLBACK_PEAKS)
    peaks = {"hbm_gbs": hbm, "bf16_tflops": flops, "source": "measured"}
    sustained = _number_under(raw, "bf16_tflops_sustained")
    if sustained:
        peaks["bf16_tflops_sustained"] = sustained
    return peaks


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.proc, self.index = [], None, index
        self.times, self.regions = [], []          # when each sample was read; (name, start, stop) of the timed regions

    def region(self, name, start, stop):
        self.regions.append((name, start, stop))

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)
                self.times.append(time.time())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = [int(s[0]) for s in self.samples if s[0].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        out = {"sm_mhz": int(statistics.median(mhz)) if mhz else None,
               "sm_max_mhz": int(self.samples[0][1]) if self.samples[0][1].isdigit() else None,
               "reasons": reasons, "samples": len(self.samples)}
        # the same over the decode regions alone (the median above includes the prompt steps, which run at the power limit)
        inside = [int(s[0]) for s, t in zip(self.samples, self.times)
                  if s[0].isdigit() and any(a <= t <= b + 0.06 for name, a, b in self.regions if name == "decode")]
        if inside:
            out["sm_mhz_decode"], out["samples_decode"] = int(statistics.median(inside)), len(inside)
        return out


def unequal_lengths(n, longest, rng):
    """n prompt lengths between 3/4 of `longest` and `longest`, the longest included."""
    import numpy as np
    lengths = rng.integers(max(1, longest * 3 // 4), longest + 1, size=n)
    lengths[0] = longest
    return [int(x) for x in lengths]


def weight_bytes_per_step(cfg, layers, rows):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = ((nq + 2 * nkv) * d * H + H * nq * d + 3 * H * I) * 2 + (2 * H + 2 * d) * 4
    return layers * per_layer + V * H * 2 + H * 4 + rows * H * 2   # + lm_head, final norm, embedding rows read


def prefill_flops(cfg, layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * T * ((nq + 2 * nkv) * d * H + H * nq * d + 3 * H * I)
    attention = 2 * 2 * nq * d * (T * (T + 1) // 2)          # QK^T and PV over the causal half
    return layers * (linear + attention) + 2 * V * H          # + the one row of logits that is wanted


def decode_run(q, engine, sampler, torch, rng, batch, longest_prompt, steps, warmup, clocks=None):
    """Prefill `batch` unequal prompts in one step, then time `steps` decode steps on the device."""
    import numpy as np
    lengths = unequal_lengths(batch, longest_prompt, rng)
    slots = [engine.new_sequence() for _ in range(batch)]
    prompts = [rng.integers(0, engine.vocab_size, size=n).tolist() for n in lengths]
    # prompts go in slices so that scratch stays small; every slice is a step of unequal lengths
    chunk = max(1, 8192 // max(lengths))
    ids = torch.empty(batch, dtype=torch.int32, device=engine.device)
    for lo in range(0, batch, chunk):
        part = range(lo, min(batch, lo + chunk))
        logits = engine.step([q.StepEntry(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in part])
        ids[lo:lo + len(part)] = sampler.choose_device(logits, list(part), [0] * len(part))
    entries = [q.StepEntry(s, [0], [0]) for s in slots]
    seq_ids = list(range(batch))

    def one(step_index):
        logits = engine.step(entries, device_tokens=ids)
        ids.copy_(sampler.choose_device(logits, seq_ids, [step_index] * batch))

    t_region = time.time()
    for i in range(warmup):
        one(1 + i)
    torch.cuda.synchronize()
    launches_before = engine.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        one(1 + warmup + i)
    stop.record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.region("decode", t_region, time.time())
    ms = start.elapsed_time(stop) / steps
    cached = sum(engine.length(s) for s in slots) - batch * steps / 2.0      # mean over the timed steps
    launches = (engine.launches - launches_before) + steps                     # + the sampler's kernel
    for s in slots:
        engine.release(s)
    return {"ms": ms, "tok_s": batch / ms * 1e3, "cached_tokens": cached, "launches": launches,
            "longest": max(lengths) + warmup + steps}


E2E_SETTLE_STEPS = 40


def e2e_run(q, engine, torch, rng, batch, longest_prompt, steps, warmup, clocks=None):
    """Through `generate_token_ids`: host prompts in, host token ids out; the decode steps after
    the warm-up are timed on the host clock (each ends with the device-to-host read of its ids).

    The entry point runs all prompts of the batch as ONE step (tens of thousands of tokens at the power
    limit), after which the SM clock needs some 100 ms to come back up; decode steps in that tail run at
    the lower clock.  So the warm-up here is `warmup` + E2E_SETTLE_STEPS untimed decode steps, and the
    number is that of generation in steady state.  `host_ms` is what the host spends per step on
    launching (step + choice), not counting its wait for the ids."""
    lengths = unequal_lengths(batch, longest_prompt, rng)
    prompts = [rng.integers(0, engine.vocab_size, size=n).tolist() for n in lengths]
    warmup = warmup + E2E_SETTLE_STEPS
    marks, busy = [], [0.0, 0]

    def on_token(index, token):
        if index == 0:
            marks.append(time.perf_counter())

    real_step = engine.step

    def timed_step(*a, **k):
        t0 = time.perf_counter()
        out = real_step(*a, **k)
        if len(marks) > warmup:
            busy[0] += time.perf_counter() - t0
            busy[1] += 1
        return out

    engine.step = timed_step
    try:
        q.generate_token_ids(engine, prompts, q.SamplingParams(mode="greedy"),
                             q.GenerationOptions(max_new_tokens=1 + warmup + steps), on_token=on_token)
    finally:
        del engine.step
    torch.cuda.synchronize()
    # marks[k] is taken after step k's ids reached the host; step 0 is the prefill
    seconds = marks[warmup + steps] - marks[warmup]
    if clocks is not None:                          # the decode steps after the prompt step settled
        clocks.region("decode", time.time() - (time.perf_counter() - marks[E2E_SETTLE_STEPS // 2]), time.time())
    return {"tok_s": batch * steps / seconds, "ms": seconds / steps * 1e3, "warmup": warmup,
            "host_ms": busy[0] / max(busy[1], 1) * 1e3}


def products_against_the_vendor_library(torch, cfg, copies=6, repeats=21, token_counts=(129, 256, 512, 1024, 2048, 4096)):
    """Microseconds of Y = X . W^T for the q/k/v, output, gate/up and down projections of one layer, per token
    count: `ours` through parts.linear (the kernels the engine runs), `vendor` through torch.mm (cuBLAS).  Each
    is a CUDA graph of `copies` products over different weights (more than the L2 holds), the median of
    `repeats` replays divided by `copies`."""
    from qwen3_b200.csrc import ops
    from qwen3_b200.parts.linear import linear, tcgen05_form
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    d, nq, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    shapes = [("qkv", (nq + 2 * nkv) * d, H), ("o", H, nq * d), ("gate_up", 2 * I, H), ("down", H, I)]

    def replay_us(fn):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(repeats):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return statistics.median(times) / copies * 1e3

    out = {"config": {"hidden": H, "intermediate": I, "copies": copies, "repeats": repeats}, "rows": []}
    for M in token_counts:
        sums = [0.0, 0.0]
        for name, N, K in shapes:
            ws = [torch.randn(N, K, device="cuda").to(torch.bfloat16) for _ in range(copies)]
            x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            ours = replay_us(lambda: [linear(x, w, y) for w in ws])
            vendor = replay_us(lambda: [torch.mm(x, w.t(), out=y) for w in ws])
            out["rows"].append({"tokens": M, "product": name, "N": N, "K": K, "form": tcgen05_form(M, N, K),
                                "ours_us": round(ours, 1), "vendor_us": round(vendor, 1), "ratio": round(ours / vendor, 3)})
            sums[0] += ours
            sums[1] += vendor
            del ws
        out["rows"].append({"tokens": M, "product": "all four", "ours_us": round(sums[0], 1), "vendor_us": round(sums[1], 1),
                            "ratio": round(sums[0] / sums[1], 3)})
    out["status_word"] = ops.tcgen05_status("cuda")
    return out


def kernel_breakdown(q, engine, sampler, torch, rng, batch, context, cfg, layers):
    """Microseconds per entry point of this library's kernels in one decode step of the headline batch and in
    one prompt step of 2,048 tokens, from CUDA events around every launch."""
    from qwen3_b200.csrc import ops
    engine.use_graphs = False                       # every kernel launched by itself, so that each can be timed
    lengths = unequal_lengths(batch, context - 8, rng)
    slots = [engine.new_sequence() for _ in range(batch)]
    chunk = max(1, 8192 // max(lengths))
    for lo in range(0, batch, chunk):
        part = range(lo, min(batch, lo + chunk))
        engine.step([q.StepEntry(slots[i], rng.integers(0, engine.vocab_size, size=lengths[i]).tolist(), []) for i in part])
    entries = [q.StepEntry(s, [1], [0]) for s in slots]
    out = {"config": {"layers": layers, "batch": batch, "context": context, "prompt_tokens": PREFILL_TOKENS}}
    for _ in range(2):
        sampler.choose_device(engine.step(entries), list(range(batch)), [0] * batch)
    with ops.KernelTimer() as timer:
        sampler.choose_device(engine.step(entries), list(range(batch)), [0] * batch)
    out["decode_step_us"] = {k: [n, round(us, 1)] for k, (n, us) in sorted(timer.summary().items())}
    out["decode_step_total_us"] = round(sum(us for _, us in timer.summary().values()), 1)
    for s in slots:
        engine.release(s)
    prompt = rng.integers(0, engine.vocab_size, size=PREFILL_TOKENS).tolist()
    for rep in range(3):
        slot = engine.new_sequence()
        if rep < 2:
            engine.step([q.StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        else:
            with ops.KernelTimer() as timer:
                engine.step([q.StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        engine.release(slot)
    out["prompt_step_us"] = {k: [n, round(us, 1)] for k, (n, us) in sorted(timer.summary().items())}
    out["prompt_step_total_us"] = round(sum(us for _, us in timer.summary().values()), 1)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (both are reported)")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="model shape; 8b is the headline")
    ap.add_argument("--batch", type=int, default=None, help="default: the shape's own (8b: 8, 14b: 16, 32b: 8)")
    ap.add_argument("--context", type=int, default=None, help="default: the shape's own (8b: 4096, 14b: 8192, 32b: 16384)")
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (for profiling runs)")
    ap.add_argument("--products", action="store_true",
                    help="instead of the benchmark: the four projections of a layer at 129..4,096 tokens, this library's "
                         "kernels against the vendor library's (torch.mm), both replayed from CUDA graphs over rotating weights")
    ap.add_argument("--tokens", type=int, action="append", default=None,
                    help="with --products: only this token count (may be given several times); keeps a profiler's capture small")
    ap.add_argument("--kernels", action="store_true",
                    help="instead of the benchmark: time every kernel of one decode step and of one 2,048-token prompt step "
                         "with CUDA events (steps launched afresh, not replayed) and print the sums per entry point")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a CMake C++/CUDA project without a Python package and its src/core and "
                          "include/qwen3/core are absent from the checkout, so it neither installs nor compiles"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import numpy as np
    import torch
    import qwen3_b200 as q
    from qwen3_b200.sampling.sampler import Sampler

    cfg, CONTEXT, shape_batch = SHAPES[args.shape]
    if args.products:
        torch.cuda.set_device(0)
        counts = tuple(args.tokens) if args.tokens else (129, 256, 512, 1024, 2048, 4096)
        print(json.dumps(products_against_the_vendor_library(torch, cfg, token_counts=counts)))
        return 0
    CONTEXT = args.context or CONTEXT
    layers = args.layers or cfg["num_hidden_layers"]
    config = q.config_from_dict(dict(cfg, num_hidden_layers=layers))
    peaks = load_peaks()
    rng = np.random.default_rng(0)
    torch.cuda.set_device(0)
    batch = args.batch or shape_batch
    max_batch = batch if (args.skip_points or args.shape != "8b") else max(batch, 64)
    # the points at longer contexts (batch 8 at 2x and 4x the headline's) need longer sequences, not more pages
    with_points = not args.skip_points and args.shape == "8b"
    longest_context = 4 * CONTEXT if with_points else CONTEXT
    engine = q.Engine.from_random(config, seed=0, dtype="bfloat16", max_tokens=max_batch * CONTEXT,
                                  max_seq_len=longest_context)
    sampler = Sampler(q.SamplingParams(mode="greedy"), engine.vocab_size, engine.device)

    if args.kernels:
        print(json.dumps(kernel_breakdown(q, engine, sampler, torch, rng, batch, CONTEXT, cfg, layers)))
        return 0

    # headline: batch 8 whose longest sequence ends at the context length
    clocks = ClockSampler()
    clocks.__enter__()                    # sampled through every arm, warm-up included
    head = decode_run(q, engine, sampler, torch, rng, batch, CONTEXT - warmup - args.steps - 1, args.steps, warmup, clocks)
    step_bytes = weight_bytes_per_step(cfg, layers, batch) + head["cached_tokens"] * engine.cache.bytes_per_token()
    achieved = step_bytes / (head["ms"] * 1e-3) / 1e9
    e2e = e2e_run(q, engine, torch, rng, batch, CONTEXT - warmup - E2E_SETTLE_STEPS - args.steps - 1, args.steps, warmup, clocks)
    h2d = engine.last_upload_bytes

    points = {}
    if not args.skip_points and args.shape == "8b":
        for b in (1, 64):
            r = decode_run(q, engine, sampler, torch, rng, b, 2048, min(args.steps, 32), warmup, clocks)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            moved = weight_bytes_per_step(cfg, layers, b) + r["cached_tokens"] * engine.cache.bytes_per_token()
            points[f"decode_b{b}_hbm_frac"] = round(moved / (r["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        # a batch between the two, at the headline's context: the TMA + tcgen05 product instead of the few-row one
        r = decode_run(q, engine, sampler, torch, rng, 16, CONTEXT - warmup - min(args.steps, 32) - 1, min(args.steps, 32), warmup, clocks)
        points[f"decode_b16_context{CONTEXT}"] = round(r["tok_s"], 1)
        moved = weight_bytes_per_step(cfg, layers, 16) + r["cached_tokens"] * engine.cache.bytes_per_token()
        points[f"decode_b16_context{CONTEXT}_hbm_frac"] = round(moved / (r["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
        for factor in (2, 4):
            ctx = factor * CONTEXT
            r = decode_run(q, engine, sampler, torch, rng, batch, ctx - warmup - min(args.steps, 32) - 1, min(args.steps, 32), warmup,
                           clocks)
            points[f"decode_b{batch}_context{ctx}"] = round(r["tok_s"], 1)
            moved = weight_bytes_per_step(cfg, layers, batch) + r["cached_tokens"] * engine.cache.bytes_per_token()
            points[f"decode_b{batch}_context{ctx}_hbm_frac"] = round(moved / (r["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)

    # prefill: one prompt of 2,048 tokens in one step
    times = []
    for rep in range(2 + 3):
        slot = engine.new_sequence()
        prompt = rng.integers(0, engine.vocab_size, size=PREFILL_TOKENS).tolist()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([q.StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.release(slot)
        if rep >= 2:
            times.append(start.elapsed_time(stop))
    prefill_ms = statistics.median(times)
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    clocks.__exit__()

    line = {
        "metric": f"decode tok/s at batch {batch}, context {CONTEXT} (Qwen3-{args.shape.upper()} shape, random weights, 1 B200)",
        "value": round(head["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(head["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform-random token ids", "impl": "ours",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": layers, "layers_of_config": cfg["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
                   "seq_len": CONTEXT, "longest_context_reached": head["longest"], "parallelism": "none (1 GPU)",
                   "cache": "paged, 64 tokens a page", "l2": "a step reads every weight (GBs), far above the 126 MB L2",
                   "sampling": "greedy on the device"},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms"], 4),
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4 * batch, "warmup": e2e["warmup"],
                "host_ms_per_step": round(e2e["host_ms"], 4)},
        "gpu_launches": int(head["launches"]),
        "prefill": {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
                    # beside the burst peak: what the vendor's product keeps up for seconds under the power limit
                    **({"frac_of_sustained": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)}
                       if peaks.get("bf16_tflops_sustained") else {})},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
        "points": points,
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
