"""CPU: pins the oracle against the golden vectors (the reference's in-test math restated in
numpy by tests/golden/make_golden.py) with the tolerances the reference's tests use, and checks
the oracle's own consistency the way the reference's integration tests do."""
import numpy as np
import pytest


# ---- reference generator -------------------------------------------------------------------
def test_lcg_matches_golden(orc, golden):
    assert np.array_equal(orc.lcg(8, 1), golden["lcg_seed1_first8"])


# ---- src/nn/ops/emit.rs:1001-1006, tol 1e-3 (emit.rs:1071) -----------------------------------
@pytest.mark.parametrize("seq,heads,hd", [(8, 2, 4), (37, 3, 16), (65, 12, 64)])
def test_flash_recurrence_matches_full_softmax(orc, golden, seq, heads, hd):
    dim = heads * hd
    q = orc.lcg(seq * dim, 1).reshape(seq, dim)
    k = orc.lcg(seq * dim, 2).reshape(seq, dim)
    v = orc.lcg(seq * dim, 3).reshape(seq, dim)
    out, lse = orc.flash_attention(q, k, v, hd, with_lse=True)
    ref = golden[f"flash_{seq}_{heads}_{hd}"]
    assert np.max(np.abs(out - ref)) < 1e-3
    assert np.all(np.isfinite(lse))


# ---- src/nn/ops/emit.rs:1333-1337, tol 1e-4 (emit.rs:1417) -----------------------------------
@pytest.mark.parametrize("attn_len,heads,hd", [(1, 2, 4), (5, 3, 16), (33, 12, 64)])
def test_cached_attention_matches_golden(orc, golden, attn_len, heads, hd):
    dim, max_ctx = heads * hd, 64
    q = orc.lcg(dim, 1)
    k = orc.lcg(max_ctx * dim, 2).reshape(max_ctx, dim)
    v = orc.lcg(max_ctx * dim, 3).reshape(max_ctx, dim)
    out = orc.decode_attention(q, k, v, attn_len, hd)
    assert np.max(np.abs(out - golden[f"cached_{attn_len}_{heads}_{hd}"])) < 1e-4


# ---- src/nn/ops/emit.rs:1424-1465, tol 1e-4 --------------------------------------------------
def test_gemv_and_gemv_add_match_golden(orc, golden):
    n, k = 301, 19
    a = orc.lcg(k, 10).reshape(1, k)
    b = orc.lcg(k * n, 20).reshape(k, n)
    c0 = orc.lcg(n, 30).reshape(1, n)
    c = orc.matmul(a, b)
    c_add = orc.matmul(a, b, c0)
    # same summation order as the reference's `dot`: bit-equal, not just within 1e-4
    assert np.array_equal(c[0], golden["gemv"])
    assert np.array_equal(c_add[0], golden["gemv_add"])


def test_matmul_rows_equal_gemv_rows(orc):
    """m > 1 uses the same per-element order as m == 1 (prefill == decode arithmetic)."""
    a = orc.lcg(7 * 33, 5).reshape(7, 33)
    b = orc.lcg(33 * 130, 6).reshape(33, 130)
    full = orc.matmul(a, b)
    for i in range(7):
        assert np.array_equal(full[i], orc.matmul(a[i:i + 1], b)[0])


# ---- src/nn/ops/emit.rs:1468-1504 ------------------------------------------------------------
def test_silu_residual_probes(orc, golden):
    idx = golden["silu_probe_idx"]
    data = ((idx % 1000).astype(np.float32) - np.float32(500.0)) / np.float32(250.0)
    res = (idx % 777).astype(np.float32) / np.float32(777.0)
    got = orc.silu(data) + res
    assert np.max(np.abs(got - golden["silu_probe_expected"])) < 1e-5


# ---- src/nn/sampling.rs:95-141 ---------------------------------------------------------------
def test_greedy_kats(orc, golden):
    logits = golden["kat_logits"]
    assert orc.argmax(logits) == int(golden["kat_greedy"][0])
    assert orc.sample_greedy(logits) == 3
    assert orc.sample_greedy(logits, golden["kat_penalty_seen"], float(golden["kat_penalty_value"][0])) == \
        int(golden["kat_penalty_greedy"][0])


def test_argmax_first_maximum_wins(orc):
    assert orc.argmax(np.array([1.0, 5.0, 5.0, 2.0], np.float32)) == 1
    assert orc.argmax(np.array([-1.0, -1.0], np.float32)) == 0


# ---- kernels vs plain numpy ------------------------------------------------------------------
def test_rmsnorm_embedding_rope(orc):
    x = orc.lcg(5 * 24, 7).reshape(5, 24)
    w = orc.lcg(24, 8)
    y = orc.rmsnorm(x, w, 1e-5)
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5) * w
    assert np.max(np.abs(y - ref)) < 1e-5
    table = orc.lcg(11 * 6, 9).reshape(11, 6)
    e = orc.embedding(np.array([3, 10, 11, 4000000000], np.uint32), table)
    assert np.array_equal(e[0], table[3]) and np.array_equal(e[1], table[10])
    assert not e[2].any() and not e[3].any()  # out-of-range id -> zero row (src/shaders/cuda.rs:21-29)
    # rope: rotation preserves pair norms; position 0 is the identity; offset == shifted rows
    v = orc.lcg(6 * 16, 10).reshape(6, 16)
    r = orc.rope(v, 8)
    assert np.array_equal(r[0], v[0])
    assert np.allclose((r.reshape(6, 8, 2) ** 2).sum(-1), (v.reshape(6, 8, 2) ** 2).sum(-1), atol=1e-5)
    one = orc.rope(v[4:5], 8, pos_offset=4)
    assert np.array_equal(one[0], r[4])
    # explicit formula for one element (src/shaders/cpu.rs:98-103)
    d, hd, pos = 2, 8, 3
    freq = np.float32(1.0) / np.float32(np.power(np.float32(10000.0), np.float32(d) / np.float32(hd)))
    ang = np.float32(pos) * freq
    exp0 = v[3, d] * np.cos(ang) - v[3, d + 1] * np.sin(ang)
    assert abs(r[3, d] - exp0) < 1e-6


# ---- src/nn/inference.rs:334-359: prefill logits == sequential decode, tol 1e-3 ----------------
def _weights(ak, cfg, seed, std):
    return ak.synthetic_weights(cfg, seed=seed, std=std)


def test_prefill_logits_match_sequential_decode(ak, orc):
    cfg = ak.ModelConfig(97, 32, 4, 2, 16)
    params = _weights(ak, cfg, 42, 0.15)
    prompt = np.array([3, 41, 7, 96, 0, 25], np.uint32)
    m = orc.Model(cfg.as_dict(), params)
    s1 = orc.Session(m, 16)
    rc, pl = s1.prefill(prompt)
    assert rc == 0 and pl.shape == (97,)
    s2 = orc.Session(m, 16)
    for t in prompt:
        rc, dl = s2.decode_step(int(t))
        assert rc == 0
    assert np.max(np.abs(pl - dl)) < 1e-3
    # and the caches agree: K rows are post-RoPE, V rows raw
    for layer in range(2):
        k1, v1 = s1.cache(layer)
        k2, v2 = s2.cache(layer)
        assert np.max(np.abs(k1 - k2)) < 1e-4 and np.max(np.abs(v1 - v2)) < 1e-4


# ---- src/bin/diagnose.rs:675-743 (CHECK 9): KV-cache path == naive full forward, tol 1e-3 ------
def test_kv_cache_equals_naive_forward(ak, orc):
    cfg = ak.ModelConfig(64, 64, 4, 2, 16)
    params = _weights(ak, cfg, 7, 0.1)
    full = ak.uniform_tokens(14, 64, seed=3)
    m = orc.Model(cfg.as_dict(), params)
    s = orc.Session(m, 16)
    rc, logits = s.prefill(full[:4])
    cached = [logits]
    for t in full[4:-1]:
        rc, logits = s.decode_step(int(t))
        assert rc == 0
        cached.append(logits)
    for i, cur in enumerate(range(4, 14)):
        naive = orc.Session(m, 16)
        rc, nl = naive.prefill(full[:cur])
        assert np.max(np.abs(nl - cached[i])) < 1e-3


# ---- error contract, src/nn/inference.rs:62-75,181-185 ------------------------------------------
def test_session_error_codes(ak, orc):
    cfg = ak.ModelConfig(50, 16, 2, 1, 8)
    m = orc.Model(cfg.as_dict(), _weights(ak, cfg, 1, 0.1))
    s = orc.Session(m, 4)
    assert s.prefill(np.array([], np.uint32))[0] == 1          # EmptyPrompt
    assert s.prefill(np.arange(5, dtype=np.uint32))[0] == 2    # PromptTooLong
    assert s.prefill(np.arange(4, dtype=np.uint32))[0] == 0
    assert s.prefill(np.arange(2, dtype=np.uint32))[0] == 5    # CacheNotEmpty
    assert s.decode_step(1)[0] == 3                            # ContextFull
    s.reset()
    assert s.cur_len == 0 and s.decode_step(1)[0] == 0


def test_bf16_rounding_helper(orc):
    x = np.array([1.0, 1.00390625, 1.005859375, -2.5, 3.1415927], np.float32)
    y = orc.round_bf16(x)
    assert y[0] == 1.0 and y[3] == -2.5
    assert y[1] == 1.0            # tie to even (1 + 2^-8 is halfway between 1 and 1 + 2^-7)
    assert y[2] == np.float32(1.0078125)
    assert abs(y[4] - 3.140625) < 1e-7


def test_thread_count_does_not_change_results(ak, orc):
    cfg = ak.ModelConfig(97, 32, 4, 2, 16)
    params = _weights(ak, cfg, 5, 0.15)
    prompt = ak.uniform_tokens(9, 97, seed=2)
    m = orc.Model(cfg.as_dict(), params)
    outs = []
    for th in (1, orc.max_threads()):
        orc.set_threads(th)
        s = orc.Session(m, 16)
        st, toks, logits = s.generate_greedy(prompt, 5, want_logits=True)
        outs.append((toks.copy(), logits.copy()))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])


def test_block_pool_lowest_first(orc):
    p = orc.BlockPool(6)
    got = [p.alloc() for _ in range(4)]
    assert got == [0, 1, 2, 3]
    p.free(1)
    p.free(3)
    assert p.alloc() == 1 and p.alloc() == 3 and p.alloc() == 4 and p.alloc() == 5 and p.alloc() == -1
