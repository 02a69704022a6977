"""Byte-level BPE tokenizer read from a Hugging Face `tokenizer.json`.

What the reference implements (src/tokenizer/tokenizer.cpp:329-678 load, :761-794 decode;
src/tokenizer/tokenizer_encode.cpp:108-475 encode): vocabulary and merge ranks of a BPE
model, the GPT-2 byte <-> printable-character table (:156-198), added tokens matched first
(earliest match, longest among those that start there), NFC normalisation, the
pre-tokenizer's split pattern with gaps kept, then greedy merging of the lowest-ranked
adjacent pair.  Decoding concatenates the tokens' bytes.  The reference needs ICU for the
pattern; here the `regex` module supplies the Unicode classes.
"""
from __future__ import annotations

import json
import unicodedata
from typing import Dict, List, Tuple

import regex


def bytes_to_unicode() -> Dict[int, str]:
    """The printable stand-in of every byte: visible Latin-1 characters map to themselves, the
    rest to code points from 256 upwards."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class Tokenizer:
    def __init__(self, vocab: Dict[str, int], merges: List[Tuple[str, str]], added: Dict[str, int], pattern: str,
                 normalize_nfc: bool = True):
        self.vocab = vocab
        self.ranks = {pair: i for i, pair in enumerate(merges)}
        self.added = added
        self.pattern = regex.compile(pattern)
        self.normalize_nfc = normalize_nfc
        self.byte_to_char = bytes_to_unicode()
        self.char_to_byte = {c: b for b, c in self.byte_to_char.items()}
        self.id_to_token = {i: t for t, i in vocab.items()}
        self.id_to_added = {i: t for t, i in added.items()}
        ids = set(self.id_to_token) | set(self.id_to_added)
        self.vocab_size = max(ids) + 1 if ids else 0
        if len(ids) != self.vocab_size:
            raise ValueError("tokenizer ids are not dense")
        self._added_by_length = sorted(added, key=len, reverse=True)
        self._cache: Dict[str, List[int]] = {}

    @classmethod
    def load(cls, path: str) -> "Tokenizer":
        with open(path, "r", encoding="utf-8") as f:
            root = json.load(f)
        model = root["model"]
        if model.get("type") != "BPE":
            raise ValueError("only BPE tokenizers are supported")
        merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else (m[0], m[1]) for m in model["merges"]]
        added = {t["content"]: t["id"] for t in root.get("added_tokens", [])}
        pattern = None
        pre = root.get("pre_tokenizer") or {}
        for item in (pre.get("pretokenizers") or [pre]):
            if item.get("type") == "Split":
                pattern = item["pattern"].get("Regex") or regex.escape(item["pattern"].get("String", ""))
        if pattern is None:
            raise ValueError("the tokenizer has no Split pre-tokenizer pattern")
        nfc = (root.get("normalizer") or {}).get("type") == "NFC"
        return cls(model["vocab"], merges, added, pattern, nfc)

    # -- encode
    def _split_added(self, text: str):
        """Pieces (is_added, text): at each position the earliest added token wins, the longest
        among those that start there."""
        pieces, start, i = [], 0, 0
        while self.added and i < len(text):
            best_pos, best = len(text), None
            for token in self._added_by_length:
                pos = text.find(token, i)
                if pos != -1 and (pos < best_pos or (pos == best_pos and best is not None and len(token) > len(best))):
                    best_pos, best = pos, token
            if best is None:
                break
            if best_pos > start:
                pieces.append((False, text[start:best_pos]))
            pieces.append((True, best))
            start = i = best_pos + len(best)
        if start < len(text):
            pieces.append((False, text[start:]))
        return pieces

    def _bpe(self, word: str) -> List[int]:
        cached = self._cache.get(word)
        if cached is not None:
            return cached
        parts = list(word)
        while len(parts) > 1:
            best_rank, best_i = None, -1
            for i in range(len(parts) - 1):
                rank = self.ranks.get((parts[i], parts[i + 1]))
                if rank is not None and (best_rank is None or rank < best_rank):
                    best_rank, best_i = rank, i
            if best_rank is None:
                break
            a, b = parts[best_i], parts[best_i + 1]
            merged, i = [], 0
            while i < len(parts):          # every non-overlapping occurrence of the pair, left to right
                if i < len(parts) - 1 and parts[i] == a and parts[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        try:
            ids = [self.vocab[p] for p in parts]
        except KeyError as e:
            raise ValueError(f"piece {e.args[0]!r} is not in the vocabulary") from None
        self._cache[word] = ids
        return ids

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for is_added, piece in self._split_added(text):
            if is_added:
                ids.append(self.added[piece])
                continue
            if self.normalize_nfc:
                piece = unicodedata.normalize("NFC", piece)
            pos = 0
            for m in self.pattern.finditer(piece):
                for chunk in (piece[pos:m.start()], m.group(0)):      # a gap between matches is kept as a piece
                    if chunk:
                        ids.extend(self._bpe("".join(self.byte_to_char[b] for b in chunk.encode("utf-8"))))
                pos = m.end()
            if pos < len(piece):
                ids.extend(self._bpe("".join(self.byte_to_char[b] for b in piece[pos:].encode("utf-8"))))
        return ids

    # -- decode
    def decode(self, ids: List[int]) -> str:
        out, pending = [], bytearray()
        for i in ids:
            if i in self.id_to_added:
                out.append(pending.decode("utf-8", errors="replace"))
                pending = bytearray()
                out.append(self.id_to_added[i])
            elif i in self.id_to_token:
                pending.extend(self.char_to_byte[c] for c in self.id_to_token[i])
            else:
                raise ValueError(f"token id {i} is not in the tokenizer")
        out.append(pending.decode("utf-8", errors="replace"))
        return "".join(out)
