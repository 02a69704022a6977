"""Ways of cutting the same requests into steps, in the trace format of bin/trace_run:
    {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}
Each builder returns (steps, rows) where rows[i] lists, for step i, the (request id,
position) of every wanted logits row in output order."""


def whole(requests):
    """Each request alone, all its tokens in one step, logits at every position."""
    steps, rows = [], []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
        rows.append([(rid, p) for p in range(len(toks))])
    return steps, rows


def tail_one_by_one(requests, tail=32):
    """Each request alone: the prefix in one step, then the last `tail` tokens one a step
    (a request of at most `tail` tokens goes token by token from its first token)."""
    steps, rows = [], []
    for rid, toks in requests.items():
        cut = max(len(toks) - tail, 0)
        if cut > 0:
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:cut], "want": [cut - 1]}], "end": []})
            rows.append([(rid, cut - 1)])
        for p in range(cut, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            rows.append([(rid, p)])
    return steps, rows


def batched(requests, prompt_lengths, batch_size, want_all_prompt=False):
    """Batches of `batch_size` requests that start together: their prompts (the first
    prompt_lengths[id] tokens) in one step, then one token each per step from the request's
    own next tokens; a request whose tokens are used up ends and leaves the batch; the next
    batch starts when the last request of this one has ended."""
    steps, rows = [], []
    ids = list(requests)
    for b in range(0, len(ids), batch_size):
        group = ids[b:b + batch_size]
        fed = {}
        entries, out, end = [], [], []
        for rid in group:
            n = prompt_lengths[rid]
            want = list(range(n)) if want_all_prompt else [n - 1]
            entries.append({"id": rid, "tokens": requests[rid][:n], "want": want})
            out += [(rid, p) for p in want]
            fed[rid] = n
            if n == len(requests[rid]):
                end.append(rid)
        steps.append({"step": len(steps), "entries": entries, "end": end})
        rows.append(out)
        live = [rid for rid in group if fed[rid] < len(requests[rid])]
        while live:
            entries, out, end = [], [], []
            for rid in live:
                p = fed[rid]
                entries.append({"id": rid, "tokens": [requests[rid][p]], "want": [0]})
                out.append((rid, p))
                fed[rid] = p + 1
                if fed[rid] == len(requests[rid]):
                    end.append(rid)
            steps.append({"step": len(steps), "entries": entries, "end": end})
            rows.append(out)
            live = [rid for rid in live if fed[rid] < len(requests[rid])]
    return steps, rows


def peak_tokens(steps, page=64):
    """Most tokens live requests hold at any time, each rounded up to a multiple of `page`."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // page) * page for n in held.values()))
        for rid in s["end"]:
            del held[rid]
    return peak


def chunked(requests, cuts):
    """Each request alone, its tokens fed in several steps of more than one token: `cuts[id]` lists
    where a new step begins (so every step after the first continues a sequence at a position
    above 0 with several tokens at once); logits at every position."""
    steps, rows = [], []
    for rid, toks in requests.items():
        edges = [0] + [c for c in cuts[rid] if 0 < c < len(toks)] + [len(toks)]
        for lo, hi in zip(edges[:-1], edges[1:]):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[lo:hi], "want": list(range(hi - lo))}],
                          "end": [rid] if hi == len(toks) else []})
            rows.append([(rid, p) for p in range(lo, hi)])
    return steps, rows


def mixed(requests, first, chunk):
    """All requests together.  Step 0 brings the first `first[id]` tokens of each.  From then on every
    step brings, for each request that still has tokens, either one token (ids whose `chunk[id]` is 1)
    or up to `chunk[id]` tokens at once: steps that mix sequences going on by one token with sequences
    that continue by several.  Logits at every position."""
    steps, rows = [], []
    fed = {}
    entries, out, end = [], [], []
    for rid, toks in requests.items():
        n = min(first[rid], len(toks))
        entries.append({"id": rid, "tokens": toks[:n], "want": list(range(n))})
        out += [(rid, p) for p in range(n)]
        fed[rid] = n
        if n == len(toks):
            end.append(rid)
    steps.append({"step": 0, "entries": entries, "end": end})
    rows.append(out)
    live = [rid for rid in requests if fed[rid] < len(requests[rid])]
    while live:
        entries, out, end = [], [], []
        for rid in live:
            lo = fed[rid]
            hi = min(lo + chunk[rid], len(requests[rid]))
            entries.append({"id": rid, "tokens": requests[rid][lo:hi], "want": list(range(hi - lo))})
            out += [(rid, p) for p in range(lo, hi)]
            fed[rid] = hi
            if hi == len(requests[rid]):
                end.append(rid)
        steps.append({"step": len(steps), "entries": entries, "end": end})
        rows.append(out)
        live = [rid for rid in live if fed[rid] < len(requests[rid])]
    return steps, rows


def shrinking(live_counts, prompt_of=lambda i: 1 + i % 5):
    """Lengths for one batch whose number of live sequences in decode step k is live_counts[k]
    (non-increasing): request i has a prompt of prompt_of(i) tokens and then as many further
    tokens as there are steps with more than i live sequences.  Returns (total lengths, prompt lengths)."""
    n = live_counts[0]
    assert all(a >= b for a, b in zip(live_counts[:-1], live_counts[1:])) and live_counts[-1] >= 1
    prompts = [prompt_of(i) for i in range(n)]
    totals = [prompts[i] + sum(1 for c in live_counts if c > i) for i in range(n)]
    return totals, prompts
