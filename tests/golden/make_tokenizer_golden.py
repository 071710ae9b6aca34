#!/usr/bin/env python
"""Writes tests/golden/tokenizer_golden.json: token ids the Hugging Face `tokenizers` library (the crate the
reference's AkashaTokenizer wraps, src/tokenizer.rs:4-49) produces from the reference's tokenizer.json for a set of
sample strings written for this test, and the text it decodes them back to.

    python tests/golden/make_tokenizer_golden.py [path/to/tokenizer.json]

Needs the `tokenizers` package and the reference's tokenizer.json (the argument, else the AKASHA_TOKENIZER
environment variable, else the reference checkout's copy); only ids and strings are stored, not the vocabulary.
"""
import json
import os
import sys

SAMPLES = [
    "Hello, world!",
    "  leading spaces and   runs   of spaces  ",
    "It's the cat's toy; they're sure we've seen it, I'm told he'll say he'd go.",
    "Numbers: 0 7 42 1234567890 3.14159 1e-9 2026-11-25",
    "tabs\tand\nnewlines\r\n\n  mixed \t whitespace\n",
    "punctuation!!! ... ??? --- (parens) [brackets] {braces} <angle> \"quotes\" 'single'",
    "CamelCaseWordsAndSNAKE_case_words and kebab-case-words",
    "naïve café résumé coöperate Ångström",
    "Ελληνικά кириллица עברית العربية हिन्दी 日本語のテキスト 中文文本 한국어",
    "emoji 😀🚀👩‍💻 and symbols ©®™ ∑∫√ ≤≥≠ →←↑↓",
    "a<|endoftext|>b <|endoftext|><|endoftext|> tail",
    "x",
    "",
    " ",
    "The quick brown fox jumps over the lazy dog. " * 3,
    "def f(x):\n    return x ** 2  # square\n\nprint(f(12))\n",
    "https://example.org/path?query=1&other=two#frag user@example.org",
    " non-breaking em-space​zero-width",
]


def main():
    from tokenizers import Tokenizer
    path = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AKASHA_TOKENIZER", "/root/reference/tokenizer.json")
    tok = Tokenizer.from_file(path)
    cases = []
    for s in SAMPLES:
        ids = tok.encode(s, add_special_tokens=False).ids
        cases.append({"text": s, "ids": ids, "decoded": tok.decode(ids, skip_special_tokens=True)})
    out = {"vocab_size": tok.get_vocab_size(True), "cases": cases}
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tokenizer_golden.json")
    with open(dst, "w", encoding="utf-8") as f:
        json.dump(out, f, ensure_ascii=True, indent=0)
    print(f"wrote {dst}: {len(cases)} cases")


if __name__ == "__main__":
    main()
