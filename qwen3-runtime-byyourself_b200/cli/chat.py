"""Command line in the manner of the reference's `qwen3_chat` (apps/qwen3_chat.cpp).

Options the reference has keep their names, defaults and meaning (:71-153, :293-507):
MODEL_DIRECTORY / --model, --gpu, --max-context (4096, at most max_position_embeddings),
--max-new-tokens (512, clamped to the room left in the context), --sample / --greedy,
--temperature 0.6, --top-k 20 (at most the vocabulary), --top-p 0.95, --seed 42,
--thinking / --no-thinking, --show-thinking / --hide-thinking, --system TEXT,
--stop-token ID (repeatable, added to eos and bos).  The stop set is {eos, bos} plus
extras (:830-843); a trailing stop token is dropped from what is printed (:1018-1021).

Additions: raw token ids in and out without any tokenizer (--tokens, --tokens-file),
several prompts of unequal length as one batch, --dtype, and --random-weights SEED with
--config for a model that exists only as a configuration.  Text chat needs tokenizer.json
in the model folder.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
from typing import List, Optional

USAGE_TAIL = """
While chatting, a line that starts with a slash is a command:
  /exit, /quit   leave
  /clear         forget the conversation so far
  /think on      let the model reason before it answers
  /think off     ask for the answer straight away
  /help          this list
"""


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="qwen3_chat", description="Qwen3 dense generation on one B200.",
                                 epilog=USAGE_TAIL, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model_directory", nargs="?", metavar="MODEL_DIRECTORY",
                    help="Folder with config.json, the safetensors and (for text) tokenizer.json.")
    ap.add_argument("--model", metavar="PATH", help="The same folder, given as an option.")
    ap.add_argument("--gpu", type=int, default=0, metavar="INDEX", help="Which CUDA device to run on (default 0).")
    ap.add_argument("--max-context", type=int, default=None, metavar="TOKENS",
                    help="Longest sequence, prompt and answer together, that the cache and the rotation table are sized for "
                         "(default 4096, never more than the model's own limit).")
    ap.add_argument("--max-new-tokens", type=int, default=512, metavar="TOKENS",
                    help="Stop an answer after this many new tokens (default 512; less if the context is nearly full).")
    mode = ap.add_mutually_exclusive_group()
    mode.add_argument("--sample", dest="greedy", action="store_false",
                      help="Draw each token at random from the filtered distribution (the default).")
    mode.add_argument("--greedy", dest="greedy", action="store_true",
                      help="Take the most likely token every time; no randomness.")
    ap.set_defaults(greedy=False)
    ap.add_argument("--temperature", type=float, default=0.6, metavar="VALUE",
                    help="Logits are divided by this before drawing; above 0 (default 0.6).")
    ap.add_argument("--top-k", type=int, default=20, metavar="VALUE",
                    help="Keep only the k best candidates, ties included; 0 keeps all (default 20).")
    ap.add_argument("--top-p", type=float, default=0.95, metavar="VALUE",
                    help="Keep the smallest set of best candidates whose probability reaches p; 1.0 keeps all (default 0.95).")
    ap.add_argument("--seed", type=int, default=42, metavar="VALUE",
                    help="Seed of the random streams; the same seed repeats the same answers (default 42).")
    think = ap.add_mutually_exclusive_group()
    think.add_argument("--thinking", dest="thinking", action="store_true",
                       help="Let the model write its reasoning before the answer (the default).")
    think.add_argument("--no-thinking", dest="thinking", action="store_false",
                       help="Start the answer after an empty reasoning block, so that the model answers at once.")
    ap.set_defaults(thinking=True)
    show = ap.add_mutually_exclusive_group()
    show.add_argument("--show-thinking", dest="show_thinking", action="store_true",
                      help="Print the reasoning as well as the answer (the default).")
    show.add_argument("--hide-thinking", dest="show_thinking", action="store_false",
                      help="The model may reason, but only the answer is printed.")
    ap.set_defaults(show_thinking=True)
    ap.add_argument("--system", default="", metavar="TEXT", help="A system message put before the conversation.")
    ap.add_argument("--stop-token", type=int, action="append", default=[], metavar="ID",
                    help="One more token id that ends an answer, beside the model's own; may be given several times.")
    # additions
    ap.add_argument("--tokens", action="append", default=[], metavar="IDS",
                    help="A prompt as comma-separated token ids; repeat for a batch. Prints token ids.")
    ap.add_argument("--tokens-file", metavar="PATH", help="A file with one prompt of token ids per line.")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default=None,
                    help="Compute type. Default: the checkpoint's torch_dtype")
    ap.add_argument("--config", metavar="PATH", help="config.json for --random-weights.")
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="Run the configuration of --config with seeded random weights instead of a checkpoint.")
    return ap


def parse_ids(text: str) -> List[int]:
    ids = [int(t) for t in text.replace(",", " ").split()]
    if not ids:
        raise ValueError("an empty list of token ids")
    return ids


def main(argv: Optional[List[str]] = None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.model and args.model_directory:
        ap.error("give the model directory once: MODEL_DIRECTORY or --model")
    model_dir = args.model or args.model_directory
    if model_dir is None and args.random_weights is None:
        ap.error("a model directory is required (MODEL_DIRECTORY or --model), or --random-weights with --config")
    if args.random_weights is not None and not args.config:
        ap.error("--random-weights needs --config")
    if args.max_new_tokens < 0:
        ap.error("--max-new-tokens cannot be negative")

    import qwen3_b200 as q

    config = q.load_config(args.config if args.random_weights is not None else model_dir)
    plan = config.plan()                 # sizes and stop tokens as every architecture states them
    max_context = args.max_context if args.max_context is not None else min(4096, plan.max_positions)
    if not 0 < max_context <= plan.max_positions:
        ap.error(f"--max-context must be in 1..{plan.max_positions} (the model's longest sequence)")
    if args.top_k > plan.vocab_size:
        ap.error("--top-k exceeds the vocabulary size")
    sampling = (q.SamplingParams(mode="greedy") if args.greedy else
                q.SamplingParams(mode="sample", temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                                 seed=args.seed))
    stops = sorted({*plan.stop_token_ids, *args.stop_token})
    for s in stops:
        if not 0 <= s < plan.vocab_size:
            ap.error(f"stop token {s} is outside the vocabulary")

    prompts = [parse_ids(t) for t in args.tokens]
    if args.tokens_file:
        with open(args.tokens_file) as f:
            prompts += [parse_ids(line) for line in f if line.strip()]
    device = f"cuda:{args.gpu}"
    n_live = max(1, len(prompts))

    def make_engine():
        if args.random_weights is not None:
            return q.Engine.from_random(config, args.random_weights, dtype=args.dtype, max_tokens=n_live * max_context,
                                        max_seq_len=max_context, device=device)
        return q.Engine.from_folder(model_dir, dtype=args.dtype, max_tokens=n_live * max_context,
                                    max_seq_len=max_context, device=device)

    if prompts:
        engine = make_engine()
        room = max_context - max(len(p) for p in prompts)
        if room <= 0:
            ap.error("the prompt does not leave room in the context; raise --max-context")
        results = q.generate_token_ids(engine, prompts, sampling,
                                       q.GenerationOptions(min(args.max_new_tokens, room), stops))
        for r in results:
            print(",".join(str(t) for t in r.token_ids), f"# {r.stop_reason}")
        return 0

    tokenizer_path = os.path.join(model_dir or "", "tokenizer.json")
    if not os.path.isfile(tokenizer_path):
        ap.error("no tokenizer.json in the model folder: give prompts as token ids with --tokens")
    from .chat_template import apply_chat_template, parse_answer, split_thinking
    from .tokenizer import Tokenizer
    tokenizer = Tokenizer.load(tokenizer_path)
    if tokenizer.vocab_size > plan.vocab_size:
        ap.error("the tokenizer has more ids than the model's vocabulary")
    sampling = q.SamplingParams(**{**sampling.__dict__, "valid_vocab_size": tokenizer.vocab_size})
    engine = make_engine()
    history, thinking = [], args.thinking
    print("Type a message; /help lists the commands.")
    while True:
        try:
            line = input("> ").strip()
        except EOFError:
            break
        if not line:
            continue
        if line in ("/exit", "/quit"):
            break
        if line == "/clear":
            history = []
            continue
        if line == "/help":
            print(USAGE_TAIL)
            continue
        if line in ("/think on", "/think off"):
            thinking = line.endswith("on")
            continue
        history.append(("user", line))
        messages = ([("system", args.system)] if args.system else []) + history
        ids = tokenizer.encode(apply_chat_template(messages, True, thinking))
        room = max_context - len(ids)
        if room <= 0:
            print("[the conversation no longer fits the context; use /clear]")
            history.pop()
            continue
        # like the reference, every turn prefills the whole history into a fresh sequence (:992); a turn that
        # fails, or that ends inside the reasoning block, is taken back so that user and assistant still alternate
        # (:1036-1055, :1086-1100)
        try:
            result = q.generate_token_ids(engine, [ids], sampling,
                                          q.GenerationOptions(min(args.max_new_tokens, room), stops))[0]
        except Exception as error:            # the conversation goes on without this turn
            history.pop()
            print(f"[generation failed: {error}]", file=sys.stderr)
            continue
        out = result.token_ids[:-1] if result.stop_reason == q.STOP_TOKEN else result.token_ids
        text = tokenizer.decode(out)
        answer, _, complete = parse_answer(text)
        thought, _ = split_thinking(text)
        if not complete:
            print(f"[thinking]\n{thought}" if args.show_thinking else "[the reasoning is hidden]")
            print("[the model stopped before it gave an answer; this turn is not kept in the conversation]")
            history.pop()
            continue
        if thought and args.show_thinking:
            print(f"[thinking]\n{thought}\n[answer]")
        print(answer)
        history.append(("assistant", answer))
        if result.stop_reason == q.MAX_NEW_TOKENS:
            print("[the answer was cut at --max-new-tokens]")
    return 0


if __name__ == "__main__":
    sys.exit(main())
