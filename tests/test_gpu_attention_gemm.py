"""GPU: the fused sm_100a kernels (paged decode attention, split+RoPE+append, tcgen05 GEMM)
against the oracle / plain fp32 math, through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def host(t):
    return t.detach().float().cpu().numpy()


def build_paged(torch, orc, lens, heads, hd, dtype, seed=0, shuffle=True):
    """Contiguous per-sequence K/V [len, dim] (values ~ U[-1,1]) scattered into paged pools
    [n_blocks, heads, 16, hd] through a shuffled block table."""
    rows = len(lens)
    dim = heads * hd
    max_blocks = max(1, (max(lens) + 15) // 16)
    need = sum((l + 15) // 16 for l in lens)
    n_blocks = need + 3
    rng = np.random.default_rng(seed)
    perm = rng.permutation(n_blocks) if shuffle else np.arange(n_blocks)
    tables = np.zeros((rows, max_blocks), np.int32)
    kp = np.full((n_blocks, heads, 16, hd), np.nan, np.float32)  # unwritten slots stay NaN on purpose
    vp = np.full((n_blocks, heads, 16, hd), np.nan, np.float32)
    ks, vs = [], []
    nxt = 0
    for r, L in enumerate(lens):
        k = orc.lcg(max(L, 1) * dim, 100 + 2 * r).reshape(-1, dim)[:L]
        v = orc.lcg(max(L, 1) * dim, 101 + 2 * r).reshape(-1, dim)[:L]
        if dtype == 1:
            k, v = orc.round_bf16(k), orc.round_bf16(v)
        ks.append(k)
        vs.append(v)
        for b in range((L + 15) // 16):
            blk = int(perm[nxt]); nxt += 1
            tables[r, b] = blk
            n = min(16, L - b * 16)
            kp[blk, :, :n, :] = k[b * 16:b * 16 + n].reshape(n, heads, hd).transpose(1, 0, 2)
            vp[blk, :, :n, :] = v[b * 16:b * 16 + n].reshape(n, heads, hd).transpose(1, 0, 2)
    tdt = torch.float32 if dtype == 0 else torch.bfloat16
    return (torch.from_numpy(kp).cuda().to(tdt), torch.from_numpy(vp).cuda().to(tdt),
            torch.from_numpy(tables).cuda(), ks, vs, n_blocks, max_blocks)


def ref_decode(orc, q, ks, vs, hd):
    out = np.zeros_like(q)
    for r in range(q.shape[0]):
        L = ks[r].shape[0]
        if L:
            out[r] = orc.decode_attention(q[r].copy(), np.ascontiguousarray(ks[r]), np.ascontiguousarray(vs[r]), L, hd)
    return out


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("heads,hd,lens,n_splits", [
    (12, 64, [33], 1),                                   # the reference's (33,12,64) decode shape
    (12, 64, [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 257, 511, 512], 1),
    (12, 64, [1, 16, 17, 64, 65, 200, 512, 300], 3),     # split-KV + merge
    (3, 64, [0, 5, 0, 48], 1),                           # empty sequences give zero rows
    (16, 128, [7, 128, 129, 1000], 1),
    (16, 128, [640, 33, 4096 // 4], 4),
    (2, 64, [900], 0),                                   # library-chosen split count
    (3, 16, [5, 40], 1), (2, 4, [1, 9], 1), (4, 8, [6, 16, 33], 1),   # generic head_dim path
])
def test_attn_decode_paged(ak, orc, torch_cuda, dtype, heads, hd, lens, n_splits):
    torch = torch_cuda
    rows, dim = len(lens), heads * hd
    kp, vp, tables, ks, vs, n_blocks, max_blocks = build_paged(torch, orc, lens, heads, hd, dtype)
    q = orc.lcg(rows * dim, 7).reshape(rows, dim)
    if dtype == 1:
        q = orc.round_bf16(q)
    tdt = torch.float32 if dtype == 0 else torch.bfloat16
    dq = torch.from_numpy(q).cuda().to(tdt)
    out = torch.full((rows, dim), float("nan"), device="cuda", dtype=tdt)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    nbytes = ak.ops.attn_decode_scratch_bytes(rows, heads, hd, max_blocks, n_splits, dtype)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    ak.ops.attn_decode_paged(dq, kp, vp, tables, kv_lens, out, rows, heads, hd, max_blocks, scale, dtype,
                             n_splits, n_blocks, scratch)
    torch.cuda.synchronize()
    want = ref_decode(orc, q, ks, vs, hd)
    got = host(out)
    assert np.isfinite(got).all(), "NaN leaked from masked or unwritten cache slots"
    tol = 2e-5 if dtype == 0 else 1e-2   # bf16 output rounding: 2^-8 relative on values < 1
    assert np.max(np.abs(got - want)) < tol


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("heads,hd,lens,n_splits", [
    (12, 64, [1, 2, 15, 16, 17, 32, 33, 64, 65, 200, 511, 512, 0, 49], 1),
    (12, 64, [1, 16, 17, 65, 200, 512, 300], 3),         # the split that owns the last block appends
    (4, 128, [1, 17, 128, 129, 700], 1),
    (2, 64, [900, 33], 0),
])
def test_attn_decode_append_paged(ak, orc, torch_cuda, dtype, heads, hd, lens, n_splits):
    """Fused head split + RoPE + cache append + attention equals head_gather -> rope_offset -> cache_write ->
    attn_qk_cached -> softmax_rect -> attn_av_cached of the reference's decode graph
    (src/nn/inference_graphs.rs:385-456): the output, and the K/V rows written at the new slots."""
    torch = torch_cuda
    rows, dim = len(lens), heads * hd
    kp, vp, tables, ks, vs, n_blocks, max_blocks = build_paged(torch, orc, lens, heads, hd, dtype)
    tdt = torch.float32 if dtype == 0 else torch.bfloat16
    rnd = (lambda a: orc.round_bf16(np.ascontiguousarray(a, np.float32))) if dtype == 1 else (lambda a: np.asarray(a, np.float32))
    qkv = orc.lcg(rows * 3 * dim, 77).reshape(rows, 3 * dim)
    rope_len = max(lens) + 3
    pos = np.arange(rope_len, dtype=np.float32)[:, None]
    freq = (np.float32(1.0) / np.power(np.float32(10000.0), np.arange(0, hd, 2, dtype=np.float32) / np.float32(hd))).astype(np.float32)
    ang = (pos * freq[None, :]).astype(np.float32)
    table = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)
    q_rot = np.zeros((rows, dim), np.float32)
    for r, L in enumerate(lens):
        if L == 0:
            continue
        p = L - 1
        q_rot[r] = rnd(orc.rope(qkv[r:r + 1, :dim].copy(), hd, p)[0])
        ks[r][p] = rnd(orc.rope(qkv[r:r + 1, dim:2 * dim].copy(), hd, p)[0])     # the appended rows
        vs[r][p] = rnd(qkv[r, 2 * dim:])
        blk, w = int(tables[r, p // 16]), p % 16
        kp[blk, :, w, :] = float("nan")                                          # the kernel must write them
        vp[blk, :, w, :] = float("nan")
    out = torch.full((rows, dim), float("nan"), device="cuda", dtype=tdt)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    nbytes = ak.ops.attn_decode_scratch_bytes(rows, heads, hd, max_blocks, n_splits, dtype)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    ak.ops.attn_decode_append_paged(torch.from_numpy(qkv).cuda(), torch.from_numpy(table).cuda(), rope_len, kp, vp, tables, kv_lens, out,
                                    rows, heads, hd, max_blocks, scale, dtype, n_splits, n_blocks, scratch)
    torch.cuda.synchronize()
    want = ref_decode(orc, q_rot, ks, vs, hd)
    got, gk, gv = host(out), host(kp), host(vp)
    assert np.isfinite(got).all()
    tol = 2e-5 if dtype == 0 else 1e-2
    assert np.max(np.abs(got - want)) < tol
    for r, L in enumerate(lens):
        if L == 0:
            continue
        p = L - 1
        blk, w = int(tables[r, p // 16]), p % 16
        # f32: the table above is numpy's cos/sin of a float32 angle of up to ~500 rad, the expectation the oracle's libm
        # (a last-place difference in an angle of several hundred radians moves cos/sin by a few 1e-5); bf16: one rounding step at |x| < 2
        slot_tol = 1e-4 if dtype == 0 else 8e-3
        assert np.max(np.abs(gk[blk, :, w, :].reshape(-1) - ks[r][p])) < slot_tol
        assert np.max(np.abs(gv[blk, :, w, :].reshape(-1) - vs[r][p])) < slot_tol


def test_attn_decode_scaling_property(ak, orc, torch_cuda):
    """Size-independent property at the microbench shape family: attention output is a convex
    combination of V rows, so with V == const the output is that const, whatever K and the lengths."""
    torch = torch_cuda
    rows, heads, hd = 256, 12, 64
    lens = ak.uniform_ints(rows, 1, 512, 3).tolist()
    max_blocks = 32
    n_blocks = rows * max_blocks
    kp = (torch.rand(n_blocks, heads, 16, hd, device="cuda") * 2 - 1).bfloat16()
    vp = torch.full((n_blocks, heads, 16, hd), 0.5, device="cuda").bfloat16()
    tables = torch.arange(n_blocks, device="cuda", dtype=torch.int32).reshape(rows, max_blocks)
    q = (torch.rand(rows, heads * hd, device="cuda") * 2 - 1).bfloat16()
    out = torch.full((rows, heads * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ak.ops.attn_decode_paged(q, kp, vp, tables, kv_lens, out, rows, heads, hd, max_blocks, 0.125, 1, 1, n_blocks)
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), torch.full_like(out.float(), 0.5), atol=4e-3)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("heads,hd", [(12, 64), (2, 128), (4, 8)])
def test_rope_kv_append(ak, orc, torch_cuda, dtype, heads, hd):
    """Fused split + RoPE + paged append equals head_gather x3 -> rope_offset x2 -> cache_write x2
    of the reference graph (src/nn/inference_graphs.rs:385-426); slot indexing is exact."""
    torch = torch_cuda
    tokens, dim, n_blocks = 23, heads * hd, 9
    qkv = orc.lcg(tokens * 3 * dim, 31).reshape(tokens, 3 * dim)
    positions = (np.arange(tokens) * 5 % 97).astype(np.int32)
    slots = np.random.default_rng(1).permutation(n_blocks * 16)[:tokens].astype(np.int32)
    slots[4] = -1       # row without an append
    positions[9] = -1   # inactive row: nothing written at all
    tdt = torch.float32 if dtype == 0 else torch.bfloat16
    q_out = torch.full((tokens, dim), 7.0, device="cuda", dtype=tdt)
    kp = torch.full((n_blocks, heads, 16, hd), 9.0, device="cuda", dtype=tdt)
    vp = torch.full((n_blocks, heads, 16, hd), 9.0, device="cuda", dtype=tdt)
    ak.ops.rope_kv_append(torch.from_numpy(qkv).cuda(), torch.from_numpy(positions).cuda(),
                          torch.from_numpy(slots).cuda(), q_out, kp, vp, tokens, heads, hd, dtype)
    torch.cuda.synchronize()
    gq, gk, gv = host(q_out), host(kp), host(vp)
    written = np.zeros((n_blocks, 16), bool)
    tol = 2e-6 if dtype == 0 else 8e-3
    for t in range(tokens):
        if positions[t] < 0:
            assert (gq[t] == 7.0).all()
            continue
        q = orc.rope(qkv[t:t + 1, :dim].copy(), hd, int(positions[t]))[0]
        k = orc.rope(qkv[t:t + 1, dim:2 * dim].copy(), hd, int(positions[t]))[0]
        v = qkv[t, 2 * dim:]
        assert np.max(np.abs(gq[t] - q)) < tol * 4
        if slots[t] >= 0:
            b, w = divmod(int(slots[t]), 16)
            written[b, w] = True
            assert np.max(np.abs(gk[b, :, w, :].reshape(-1) - k)) < tol * 4
            assert np.max(np.abs(gv[b, :, w, :].reshape(-1) - v)) < tol * 4
    # every slot that was not addressed is untouched
    assert (gk.transpose(0, 2, 1, 3)[~written] == 9.0).all() and (gv.transpose(0, 2, 1, 3)[~written] == 9.0).all()


# -------------------------------------------------------------------------------- tcgen05 GEMM
def bf16_round(orc, a):
    return orc.round_bf16(np.ascontiguousarray(a, np.float32))


@pytest.mark.parametrize("m,n,k", [(64, 2304, 768), (1, 768, 768), (64, 768, 3072), (7, 50257, 768), (128, 256, 64), (64, 3072, 768), (64, 8192, 2048), (100, 2048, 8192), (3, 40, 1024),
                                   (300, 520, 200), (1000, 3072, 768), (129, 24, 8), (64, 6144, 2048),
                                   # activation boxes of 16 / 32 / 64 rows (the ring's activation slots shrink with them), with a K
                                   # range that fits the ring and one that wraps it
                                   (16, 3072, 768), (20, 768, 3072), (40, 2304, 768), (20, 512, 8192), (48, 1024, 16384),
                                   # m >= 1024: the CTA-pair (cta_group::2) kernel, incl. ragged last tiles in m, n and k
                                   (1024, 256, 64), (2048, 2304, 768), (1500, 520, 200), (4096, 3072, 768), (1025, 257, 72), (20000, 768, 3072)])
def test_gemm_bf16_store_f32(ak, orc, torch_cuda, m, n, k):
    torch = torch_cuda
    a = bf16_round(orc, orc.lcg(m * k, 1).reshape(m, k))
    w = bf16_round(orc, (orc.lcg(k * n, 2) * np.float32(0.25)).reshape(k, n))   # reference layout [k, n]
    da = torch.from_numpy(a).cuda().bfloat16()
    wt = torch.empty(n, k, device="cuda", dtype=torch.bfloat16)
    ak.ops.transpose_to_bf16(torch.from_numpy(w).cuda(), wt, k, n)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
    ak.ops.gemm_bf16(da, wt, c, m, n, k, ak.EPI_STORE_F32)
    torch.cuda.synchronize()
    assert np.array_equal(host(wt), w.T)          # the transpose is exact
    want = a.astype(np.float64) @ w.astype(np.float64)
    got = host(c)
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - want)) < 1e-4 * np.sqrt(k) + 1e-5


@pytest.mark.parametrize("epi", [0, 2])
@pytest.mark.parametrize("m,n,k,ldc", [(300, 1001, 256, 1008), (64, 50257, 768, 50264), (130, 520, 200, 523), (1000, 333, 64, 336)])
def test_gemm_bf16_padded_row_pitch(ak, orc, torch_cuda, epi, m, n, k, ldc):
    """An output with a row pitch wider than n (the way to give an odd-width result vector stores): the n
    columns hold the product, the padding columns are left untouched."""
    torch = torch_cuda
    a = bf16_round(orc, orc.lcg(m * k, 3).reshape(m, k))
    w = bf16_round(orc, (orc.lcg(k * n, 4) * np.float32(0.25)).reshape(k, n))
    da = torch.from_numpy(a).cuda().bfloat16()
    wt = torch.from_numpy(np.ascontiguousarray(w.T)).cuda().bfloat16()
    cdt = torch.float32 if epi == 0 else torch.bfloat16
    c = torch.full((m, ldc), 7.0, device="cuda", dtype=cdt)
    ak.ops.gemm_bf16(da, wt, c, m, n, k, epi, ldc=ldc)
    torch.cuda.synchronize()
    got = host(c)
    want = a.astype(np.float64) @ w.astype(np.float64)
    assert (got[:, n:] == 7.0).all(), "padding columns were written"
    tol = 1e-4 * np.sqrt(k) + 1e-5 if epi == 0 else 2e-2 * max(1.0, float(np.abs(want).max()))
    assert np.max(np.abs(got[:, :n] - want)) < tol


@pytest.mark.parametrize("epi", [1, 2, 3])
@pytest.mark.parametrize("m,n,k", [(64, 768, 768), (200, 3072, 768), (33, 100, 72), (1100, 1000, 328)])
def test_gemm_bf16_epilogues(ak, orc, torch_cuda, epi, m, n, k):
    torch = torch_cuda
    a = bf16_round(orc, orc.lcg(m * k, 3).reshape(m, k))
    w = bf16_round(orc, (orc.lcg(k * n, 4) * np.float32(0.2)).reshape(k, n))
    c0 = orc.lcg(m * n, 5).reshape(m, n)
    da = torch.from_numpy(a).cuda().bfloat16()
    wt = torch.from_numpy(np.ascontiguousarray(w.T)).cuda().bfloat16()
    acc = a.astype(np.float64) @ w.astype(np.float64)
    if epi == ak.EPI_ADD_F32:
        c = torch.from_numpy(c0).cuda()
        want, tol = c0 + acc, 1e-4 * np.sqrt(k) + 1e-5
    else:
        c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
        want = acc if epi == ak.EPI_STORE_BF16 else acc / (1.0 + np.exp(-acc))
        tol = 2.0 ** -8 * max(1.0, np.abs(want).max()) + 1e-3
    ak.ops.gemm_bf16(da, wt, c, m, n, k, epi)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(c) - want)) < tol


def ref_prefill(orc, q, k, v, hd):
    """Causal attention of one sequence (q/k/v [L, dim]) with the oracle's flash attention."""
    return orc.flash_attention(np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v), hd)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("heads,hd,lens", [
    (12, 64, [33]),                                        # the reference's flash-attention test length
    (12, 64, [1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 232, 448]),
    (2, 64, [700, 3, 0, 257]),                             # several 128-query tiles, an empty sequence
    (16, 128, [5, 130, 300]),
    (2, 128, [1000]),
    (4, 8, [6, 33]),                                       # generic head_dim path
])
def test_attn_prefill_paged(ak, orc, torch_cuda, dtype, heads, hd, lens):
    """Ragged causal prefill attention over the paged pools (bf16 head_dim 64/128: the tcgen05 kernel)."""
    torch = torch_cuda
    dim = heads * hd
    kp, vp, tables, ks, vs, n_blocks, max_blocks = build_paged(torch, orc, lens, heads, hd, dtype, seed=5)
    cu = np.zeros(len(lens) + 1, np.int32)
    cu[1:] = np.cumsum(lens)
    total = int(cu[-1])
    q = orc.lcg(total * dim, 11).reshape(total, dim) * 2.0
    if dtype == 1:
        q = orc.round_bf16(q)
    tdt = torch.float32 if dtype == 0 else torch.bfloat16
    q_rows = total + 5                                     # rows past the batch stay untouched
    dq = torch.zeros(q_rows, dim, device="cuda", dtype=tdt)
    dq[:total] = torch.from_numpy(q).cuda().to(tdt)
    out = torch.full((q_rows, dim), float("nan"), device="cuda", dtype=tdt)
    seq_slot = torch.arange(len(lens), dtype=torch.int32, device="cuda")
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    ak.ops.attn_prefill_paged(dq, kp, vp, tables, max_blocks, torch.from_numpy(cu).cuda(), seq_slot, out, len(lens), max(lens),
                              q_rows, heads, hd, scale, dtype, n_blocks)
    torch.cuda.synchronize()
    ak.check(ak.lib().ak_check_device_status(None))
    got = host(out)
    assert np.isnan(got[total:]).all(), "rows outside the batch were written"
    tol = 3e-5 if dtype == 0 else 1.2e-2   # bf16: P and the output are rounded to 8 bits of mantissa
    for i, L in enumerate(lens):
        if L == 0:
            continue
        want = ref_prefill(orc, q[cu[i]:cu[i + 1]], ks[i], vs[i], hd)
        g = got[cu[i]:cu[i + 1]]
        assert np.isfinite(g).all(), "NaN leaked from masked or unwritten cache slots"
        assert np.max(np.abs(g - want)) < tol, (i, L)
