"""CPU: pins the oracle to OUTPUTS OF THE REFERENCE'S OWN KERNEL CODE.

tests/golden/reference_kernels.npz was written by `python oracle/make_ref.py --fixtures`, which
compiles the CUDA C kernel strings of the reference's src/shaders/cuda.rs, unchanged, behind a
small host shim (oracle/cuda_host_shim.h) and runs them on the reference's test shapes plus one
162M-shaped slice per kernel. Inputs are rebuilt here from the same seeds with the reference's
test generator (src/nn/ops/emit.rs:910-921); only outputs are stored. Every oracle kernel
(oracle/akasha_oracle.c, which restates the reference's CPU kernels src/shaders/cpu.rs) is held
to them: bit-exact where the two loops add in the same order, within a few float roundings where
they do not (the CUDA rmsnorm sums through a 256-thread tree, the CPU one serially).
When the reference sources are present the fixtures are also regenerated and compared, so a stale
file cannot pass.
"""
import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_make_ref():
    spec = importlib.util.spec_from_file_location("_akasha_make_ref", os.path.join(ROOT, "oracle", "make_ref.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["_akasha_make_ref"] = mod
    spec.loader.exec_module(mod)
    return mod


mr = _load_make_ref()


@pytest.fixture(scope="module")
def fx():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_kernels.npz"))


def scale_of(hd):
    return float(np.float32(1.0) / np.sqrt(np.float32(hd)))


@pytest.mark.parametrize("vocab,dim", [(97, 32), (5003, 768)])
def test_embedding(orc, fx, vocab, dim):
    table = orc.lcg(vocab * dim, 40).reshape(vocab, dim)
    toks = np.array([3, 41, 7, vocab - 1, 0, 25, vocab, 4_000_000_000], np.uint32)
    want = fx[f"embedding_{vocab}_{dim}"]
    assert np.array_equal(orc.embedding(toks, table), want)
    assert (want[-2:] == 0).all()          # out-of-range ids write zeros (src/shaders/cuda.rs:21-29)


def test_silu(orc, fx):
    assert np.array_equal(orc.silu(orc.lcg(1000, 60) * 6.0), fx["silu_1000"])
    # the reference's large-grid case (src/nn/ops/emit.rs:1468-1504): 17,000,003 elements, probes around 65535*256
    got = orc.silu(mr.silu_large_input())[mr.SILU_PROBES]
    assert np.array_equal(got, fx["silu_large_probes"])


@pytest.mark.parametrize("seq,dim,hd", mr.ROPE_SHAPES)
def test_rope(orc, fx, seq, dim, hd):
    got = orc.rope(orc.lcg(seq * dim, 10).reshape(seq, dim), hd)
    assert np.array_equal(got, fx[f"rope_{seq}_{dim}_{hd}"])


@pytest.mark.parametrize("dim,hd,pos", mr.ROPE_OFFSET_SHAPES)
def test_rope_offset(orc, fx, dim, hd, pos):
    got = orc.rope(orc.lcg(dim, 20).reshape(1, dim), hd, pos)
    assert np.array_equal(got, fx[f"rope_offset_{dim}_{hd}_{pos}"])


@pytest.mark.parametrize("seq,dim", mr.SPLIT_SHAPES)
def test_head_gather(orc, fx, seq, dim):
    qkv = orc.lcg(seq * 3 * dim, 50).reshape(seq, 3 * dim)
    for part in range(3):
        assert np.array_equal(orc.head_gather(qkv, seq, 3 * dim, dim, part * dim), fx[f"head_gather_{seq}_{dim}_{part}"])


def test_cache_write(orc, fx):
    cache = orc.lcg(16 * 48, 70).reshape(16, 48).copy()
    orc.cache_write(orc.lcg(3 * 48, 71).reshape(3, 48), cache, 5)
    assert np.array_equal(cache, fx["cache_write_3_48_5"])


@pytest.mark.parametrize("L,heads,hd", mr.ATTN_SHAPES)
def test_cached_attention_chain(orc, fx, L, heads, hd):
    dim, cap = heads * hd, max(64, L)
    q = orc.lcg(dim, 1)
    kc, vc = orc.lcg(cap * dim, 2).reshape(cap, dim), orc.lcg(cap * dim, 3).reshape(cap, dim)
    s = orc.attn_qk_cached(q, kc, L, hd)
    assert np.array_equal(s, fx[f"attn_qk_{L}_{heads}_{hd}"])
    p = orc.softmax_rect(s, scale_of(hd))
    assert np.array_equal(p, fx[f"attn_softmax_{L}_{heads}_{hd}"])
    o = orc.attn_av_cached(p, vc, hd)
    assert np.array_equal(o, fx[f"attn_av_{L}_{heads}_{hd}"])


@pytest.mark.parametrize("rows,size", mr.RMSNORM_SHAPES)
def test_rmsnorm(orc, fx, rows, size):
    x = orc.lcg(rows * size, 80).reshape(rows, size) * 3.0
    w = 1.0 + 0.1 * orc.lcg(size, 81)
    want = fx[f"rmsnorm_{rows}_{size}"]
    got = orc.rmsnorm(x, w, 1e-5)
    # the CUDA kernel adds the squares through a 256-thread tree, the CPU kernel (and the oracle) serially
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) < 2e-6


@pytest.mark.parametrize("seq,heads,hd", mr.FLASH_SHAPES)
def test_flash_attention(orc, fx, seq, heads, hd):
    dim = heads * hd
    q, k, v = (orc.lcg(seq * dim, s).reshape(seq, dim) for s in (1, 2, 3))
    out, lse = orc.flash_attention(q, k, v, hd, scale_of(hd), with_lse=True)
    assert np.array_equal(out, fx[f"flash_out_{seq}_{heads}_{hd}"])
    assert np.max(np.abs(lse - fx[f"flash_lse_{seq}_{heads}_{hd}"])) < 1e-6


def test_fixtures_are_what_the_reference_sources_produce(tmp_path, fx):
    """Where the reference sources are available, rebuild the kernels from them and regenerate every
    fixture: the committed file must be exactly what they produce."""
    ref = mr.ref_dir()
    if not os.path.exists(os.path.join(ref, "src", "shaders", "cuda.rs")):
        pytest.skip("reference sources not present on this machine")
    mr.build(ref, cuda=False)
    fresh = mr.generate_fixtures(str(tmp_path / "regen.npz"))
    assert sorted(fresh) == sorted(fx.files)
    for k in fx.files:
        assert np.array_equal(fresh[k], fx[k]), k
