"""CPU: the GPT-2 byte-level BPE tokenizer (`akasha-core_b200/tokenizer.py`), the text front/back end
of the reference's `--chat` (src/tokenizer.rs:4-49).

Two layers. (1) A tiny tokenizer.json written here exercises every step of the algorithm with answers
that can be worked out by hand. (2) Where the reference's tokenizer.json is available
(the AKASHA_TOKENIZER environment variable, else the reference checkout's copy), the implementation is held to
tests/golden/tokenizer_golden.json: ids and round-trip text that the Hugging Face `tokenizers` library
(the crate the reference wraps) produced from that file for the sample strings of
tests/golden/make_tokenizer_golden.py.
"""
import json
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def T(ak):
    import importlib
    return importlib.import_module("akasha_core_b200.tokenizer")


def tiny_spec(T):
    b2c = T._byte_table()
    base = [b2c[b] for b in range(256)]
    vocab = {c: i for i, c in enumerate(base)}
    G = b2c[ord(" ")]
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), (G, "w"), (G + "w", "o")]
    for a, b in merges:
        vocab[a + b] = len(vocab)
    return {"model": {"type": "BPE", "vocab": vocab, "merges": [f"{a} {b}" for a, b in merges]},
            "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "use_regex": True},
            "added_tokens": [{"id": len(vocab), "content": "<|endoftext|>", "special": True}]}, vocab, G


def test_tiny_bpe_by_hand(T):
    spec, vocab, G = tiny_spec(T)
    tok = T.AkashaTokenizer(spec)
    assert tok.vocab_size() == len(vocab) + 1
    # "hello" -> h e l l o -> he l l o -> he ll o -> hell o -> hello
    assert tok.encode("hello") == [vocab["hello"]]
    # " world": the space travels with the word; merges give "Ġwo" r l d
    assert tok.encode("hello world") == [vocab["hello"], vocab[G + "wo"], vocab["r"], vocab["l"], vocab["d"]]
    # lowest rank first, not leftmost first: "lhe" -> l he
    assert tok.encode("lhe") == [vocab["l"], vocab["he"]]
    # the added token is cut out before pre-tokenization and is skipped by decode
    eot = len(vocab)
    assert tok.encode("hello<|endoftext|>hello") == [vocab["hello"], eot, vocab["hello"]]
    assert tok.decode([vocab["hello"], eot, vocab[G + "wo"]]) == "hello wo"
    # bytes outside ASCII go through the stand-in table and come back as UTF-8
    ids = tok.encode("é😀")
    assert len(ids) == len("é😀".encode("utf-8")) and tok.decode(ids) == "é😀"
    assert tok.encode("") == [] and tok.decode([]) == ""
    assert tok.encode_batch(["hello", "lhe"]) == [tok.encode("hello"), tok.encode("lhe")]


def test_from_pretrained_reads_env(T, tmp_path, monkeypatch):
    spec, vocab, _ = tiny_spec(T)
    p = tmp_path / "tok.json"
    p.write_text(json.dumps(spec), encoding="utf-8")
    monkeypatch.setenv("AKASHA_TOKENIZER", str(p))
    assert T.AkashaTokenizer.from_pretrained().encode("hello") == [vocab["hello"]]
    monkeypatch.setenv("AKASHA_TOKENIZER", str(tmp_path / "missing.json"))
    with pytest.raises(FileNotFoundError):
        T.AkashaTokenizer.from_pretrained()


def test_matches_reference_tokenizer_golden(T):
    path = os.environ.get("AKASHA_TOKENIZER", "/root/reference/tokenizer.json")
    if not os.path.exists(path):
        pytest.skip("the reference's tokenizer.json is not on this machine")
    tok = T.AkashaTokenizer.from_file(path)
    golden = json.load(open(os.path.join(ROOT, "tests", "golden", "tokenizer_golden.json"), encoding="utf-8"))
    assert tok.vocab_size() == golden["vocab_size"] == 50257
    for c in golden["cases"]:
        assert tok.encode(c["text"]) == c["ids"], c["text"]
        assert tok.decode(c["ids"]) == c["decoded"], c["text"]
