"""GPT-2 byte-level BPE front/back end: the text side of `--chat` (src/main.rs:131-170).

Mirror of the reference's `AkashaTokenizer` (src/tokenizer.rs:8-49), which wraps the Hugging Face
`tokenizers` crate: `from_pretrained()` reads the `tokenizer.json` named by $AKASHA_TOKENIZER
(default "tokenizer.json" in the working directory), `encode(text)` adds no special tokens,
`decode(ids)` skips special tokens, `vocab_size()` counts the added tokens. This file implements
the algorithm that JSON describes, in plain Python on the host (token ids are the device path's
input and output; tokenising is string work):

  1. added tokens (`<|endoftext|>`) are cut out of the text first and map straight to their ids;
  2. ByteLevel pre-tokenizer with `use_regex`: the GPT-2 split pattern, no prefix space;
  3. every UTF-8 byte of a piece is mapped to a printable stand-in character (the GPT-2 byte table);
  4. BPE: repeatedly merge the adjacent pair with the lowest merge rank;
  5. decode: ids -> stand-in characters -> bytes -> UTF-8 (invalid sequences become U+FFFD).

The file itself is not shipped: point the loader at the reference's `tokenizer.json` (or any GPT-2 style
byte-level BPE file in the same JSON layout).
"""
from __future__ import annotations

import json
import os
from functools import lru_cache

import regex

# the GPT-2 pre-tokenization pattern (contractions, letters, numbers, other symbols, whitespace runs)
_SPLIT = regex.compile(r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""")


@lru_cache(maxsize=1)
def _byte_table():
    """byte value -> stand-in character: printable Latin-1 bytes map to themselves, the other 68
    bytes to code points 256, 257, ... in byte order."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class AkashaTokenizer:
    """`AkashaTokenizer` of the reference (src/tokenizer.rs:4-49)."""

    def __init__(self, spec: dict):
        model = spec["model"]
        if model.get("type") != "BPE":
            raise ValueError("tokenizer.json: only byte-level BPE models are supported")
        pre = spec.get("pre_tokenizer") or {}
        if pre.get("type") != "ByteLevel":
            raise ValueError("tokenizer.json: a ByteLevel pre-tokenizer is required")
        self.add_prefix_space = bool(pre.get("add_prefix_space", False))
        self.vocab = dict(model["vocab"])
        self.ranks = {}
        for i, m in enumerate(model["merges"]):
            a, b = m.split(" ") if isinstance(m, str) else m
            self.ranks[(a, b)] = i
        self.added = {t["content"]: int(t["id"]) for t in spec.get("added_tokens", [])}
        self.special_ids = {int(t["id"]) for t in spec.get("added_tokens", []) if t.get("special")}
        self.inverse = {i: s for s, i in self.vocab.items()}
        for s, i in self.added.items():
            self.inverse.setdefault(i, s)
        self._b2c = _byte_table()
        self._c2b = {c: b for b, c in self._b2c.items()}
        self._cache = {}
        self._added_re = regex.compile("|".join(regex.escape(s) for s in sorted(self.added, key=len, reverse=True))) if self.added else None

    # ---- construction -------------------------------------------------------------------------
    @classmethod
    def from_file(cls, path: str) -> "AkashaTokenizer":
        with open(path, encoding="utf-8") as f:
            return cls(json.load(f))

    @classmethod
    def from_pretrained(cls) -> "AkashaTokenizer":
        """$AKASHA_TOKENIZER, else ./tokenizer.json (src/tokenizer.rs:9-16). There is no download path."""
        local = os.environ.get("AKASHA_TOKENIZER", "tokenizer.json")
        if not os.path.exists(local):
            raise FileNotFoundError(f"tokenizer file `{local}` not found: provide tokenizer.json or set AKASHA_TOKENIZER")
        return cls.from_file(local)

    # ---- BPE ----------------------------------------------------------------------------------
    def _bpe(self, piece: str):
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        word = list(piece)
        while len(word) > 1:
            best, best_rank = -1, None
            for i in range(len(word) - 1):
                r = self.ranks.get((word[i], word[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best < 0:
                break
            a, b = word[best], word[best + 1]
            merged, i = [], 0
            while i < len(word):          # merge every occurrence of the best pair, left to right
                if i < len(word) - 1 and word[i] == a and word[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(word[i])
                    i += 1
            word = merged
        ids = [self.vocab[t] for t in word if t in self.vocab]
        if len(self._cache) < 1 << 16:
            self._cache[piece] = ids
        return ids

    def _encode_plain(self, text: str, out: list, first: bool):
        if self.add_prefix_space and first and text and not text[0].isspace():
            text = " " + text
        for piece in _SPLIT.findall(text):
            out.extend(self._bpe("".join(self._b2c[b] for b in piece.encode("utf-8"))))

    # ---- API (src/tokenizer.rs:27-48) -----------------------------------------------------------
    def encode(self, text: str) -> list:
        """Token ids of `text`; no special tokens are added (`encode(text, false)`)."""
        out, pos, first = [], 0, True
        if self._added_re is not None:
            for m in self._added_re.finditer(text):
                if m.start() > pos:
                    self._encode_plain(text[pos:m.start()], out, first)
                out.append(self.added[m.group(0)])
                pos, first = m.end(), False
        if pos < len(text):
            self._encode_plain(text[pos:], out, first)
        return out

    def encode_batch(self, texts) -> list:
        return [self.encode(t) for t in texts]

    def decode(self, ids) -> str:
        """Text of `ids`, special tokens skipped (`decode(ids, true)`); unknown ids are ignored."""
        data = bytearray()
        for i in ids:
            i = int(i)
            if i in self.special_ids:
                continue
            s = self.inverse.get(i)
            if s is None:
                continue
            for ch in s:
                b = self._c2b.get(ch)
                if b is None:
                    data.extend(ch.encode("utf-8"))
                else:
                    data.append(b)
        return data.decode("utf-8", errors="replace")

    def vocab_size(self) -> int:
        """Vocabulary size including added tokens (`get_vocab_size(true)`)."""
        return len(set(self.vocab.values()) | set(self.added.values()))
