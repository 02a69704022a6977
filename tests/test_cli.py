"""The command line's pieces that need no GPU: chat template, tokenizer, argument meanings."""
import json

import pytest

from qwen3_b200.cli.chat import build_parser, parse_ids
from qwen3_b200.cli.chat_template import apply_chat_template, parse_answer, split_thinking
from qwen3_b200.cli.tokenizer import Tokenizer, bytes_to_unicode

PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
           r"|\s+(?!\S)|\s+")


def test_chat_template_strings():
    # the strings of the reference's tests/unit/chat_template_test.cpp
    text = apply_chat_template([("system", "Be brief."), ("user", "Hi")])
    assert text == "<|im_start|>system\nBe brief.<|im_end|>\n<|im_start|>user\nHi<|im_end|>\n<|im_start|>assistant\n"
    text = apply_chat_template([("user", "Hi")], enable_thinking=False)
    assert text.endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    text = apply_chat_template([("user", "a"), ("assistant", "b")], add_generation_prompt=False)
    assert text == "<|im_start|>user\na<|im_end|>\n<|im_start|>assistant\nb<|im_end|>\n"
    for bad in ([], [("system", "x")], [("assistant", "x")], [("user", "a"), ("user", "b")],
                [("user", "a"), ("system", "b")], [("user", "a"), ("assistant", "b")]):
        with pytest.raises(ValueError):
            apply_chat_template(bad)
    assert split_thinking("<think>\nhm\n</think>\n\nyes") == ("hm", "yes")
    assert split_thinking("plain") == ("", "plain")
    assert split_thinking("hm</think>\n\nyes") == ("hm", "yes")
    # the reference's reading of a raw response (apps/qwen3_chat.cpp:593-643)
    assert parse_answer("<think>a</think>\n\r\nyes\n") == ("yes\n", True, True)
    assert parse_answer("<think>a</think>b</think>\nc") == ("c", True, True)          # the last closing tag counts
    assert parse_answer("<think>still going") == ("", True, False)                    # stopped inside the reasoning
    assert parse_answer("no tags") == ("no tags", False, True)
    assert split_thinking("<think>still going") == ("still going", "")
    assert split_thinking("<think>a</think>b</think>\nc") == ("a</think>b", "c")


def make_tokenizer(tmp_path):
    table = bytes_to_unicode()
    vocab = {table[b]: b for b in range(256)}
    merges = []

    def merge(a, b):
        merges.append(f"{a} {b}")
        vocab[a + b] = len(vocab)

    sp = table[ord(" ")]
    merge("l", "l"); merge("h", "e"); merge("he", "ll"); merge("hell", "o"); merge(sp, "w"); merge("o", "r")
    merge(sp + "w", "or"); merge(sp + "wor", "l"); merge(sp + "worl", "d")
    n = len(vocab)
    root = {"model": {"type": "BPE", "vocab": vocab, "merges": merges},
            "added_tokens": [{"id": n, "content": "<|im_start|>"}, {"id": n + 1, "content": "<|im_end|>"},
                             {"id": n + 2, "content": "<|im_start|>x"}],
            "normalizer": {"type": "NFC"},
            "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
                {"type": "Split", "pattern": {"Regex": PATTERN}, "behavior": "Isolated"}, {"type": "ByteLevel"}]}}
    path = tmp_path / "tokenizer.json"
    path.write_text(json.dumps(root))
    return Tokenizer.load(str(path)), vocab, n


def test_tokenizer_merges_added_tokens_and_round_trip(tmp_path):
    tok, vocab, n = make_tokenizer(tmp_path)
    assert tok.vocab_size == n + 3
    sp = bytes_to_unicode()[ord(" ")]
    assert tok.encode("hello world") == [vocab["hello"], vocab[sp + "world"]]
    assert tok.encode("hell") == [vocab["hell"]]
    # added tokens are matched first; the longest of those that start at the same place wins
    assert tok.encode("<|im_start|>hello<|im_end|>") == [n, vocab["hello"], n + 1]
    assert tok.encode("<|im_start|>x")[0] == n + 2
    for text in ("hello world", "héllo wörld\n\n  x", "日本語 テキスト 123", "<|im_start|>user\nhi<|im_end|>\n", "a  b\t c"):
        assert tok.decode(tok.encode(text)) == text
    # NFC: the decomposed and the composed spelling give the same ids
    assert tok.encode("é") == tok.encode("é")
    with pytest.raises(ValueError):
        tok.decode([n + 50])


def test_argument_names_and_defaults_follow_the_reference():
    args = build_parser().parse_args(["/models/x"])
    assert (args.model_directory, args.gpu, args.max_context, args.max_new_tokens) == ("/models/x", 0, None, 512)
    assert (args.greedy, args.temperature, args.top_k, args.top_p, args.seed) == (False, 0.6, 20, 0.95, 42)
    assert (args.thinking, args.show_thinking, args.system, args.stop_token) == (True, True, "", [])
    args = build_parser().parse_args(["--model", "m", "--greedy", "--no-thinking", "--hide-thinking", "--stop-token", "5",
                                      "--stop-token", "9", "--max-context", "128", "--tokens", "1,2,3", "--tokens", "4 5"])
    assert args.model == "m" and args.greedy and not args.thinking and not args.show_thinking
    assert args.stop_token == [5, 9] and args.max_context == 128
    assert [parse_ids(t) for t in args.tokens] == [[1, 2, 3], [4, 5]]
    with pytest.raises(SystemExit):
        build_parser().parse_args(["m", "--sample", "--greedy"])
    with pytest.raises(ValueError):
        parse_ids(" , ")
