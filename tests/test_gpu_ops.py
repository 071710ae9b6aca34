"""GPU: emitter-level kernels through the C ABI against the oracle, on the reference's own test
shapes and seeds (src/nn/ops/emit.rs:1001-1006, 1333-1337, 1424-1465, 1468-1504). Output buffers
are pre-filled with NaN: a kernel that leaves an element unwritten fails (the output-contract
canary the reference's authors plan, ARCHITECTURE.md:488-490)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def nan_like(torch, *shape):
    return torch.full(shape, float("nan"), dtype=torch.float32, device="cuda")


def host(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("seq,heads,hd", [(8, 2, 4), (37, 3, 16), (65, 12, 64), (130, 2, 128), (200, 3, 64)])
def test_flash_attention_emitter(ak, orc, golden, torch_cuda, seq, heads, hd):
    torch = torch_cuda
    dim = heads * hd
    q = orc.lcg(seq * dim, 1).reshape(seq, dim)
    k = orc.lcg(seq * dim, 2).reshape(seq, dim)
    v = orc.lcg(seq * dim, 3).reshape(seq, dim)
    out = nan_like(torch, seq, dim)
    lse = nan_like(torch, seq, heads)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    ak.ops.flash_attention(dev(torch, q), dev(torch, k), dev(torch, v), out, seq, dim, hd, scale, 0, lse)
    torch.cuda.synchronize()
    want, want_lse = orc.flash_attention(q, k, v, hd, with_lse=True)
    assert np.max(np.abs(host(out) - want)) < 1e-4
    assert np.max(np.abs(host(lse) - want_lse)) < 1e-4
    key = f"flash_{seq}_{heads}_{hd}"
    if key in golden.files:
        assert np.max(np.abs(host(out) - golden[key])) < 1e-3  # the reference's own tolerance


def test_flash_attention_row_offset(ak, orc, torch_cuda):
    """row_offset selects one batch row of a [batch*seq, dim] buffer (src/shaders/cuda.rs:651)."""
    torch = torch_cuda
    seq, heads, hd = 33, 2, 64
    dim = heads * hd
    q = orc.lcg(2 * seq * dim, 11).reshape(2 * seq, dim)
    k = orc.lcg(2 * seq * dim, 12).reshape(2 * seq, dim)
    v = orc.lcg(2 * seq * dim, 13).reshape(2 * seq, dim)
    out = nan_like(torch, 2 * seq, dim)
    scale = 0.125
    for b in range(2):
        ak.ops.flash_attention(dev(torch, q), dev(torch, k), dev(torch, v), out, seq, dim, hd, scale, b * seq)
    torch.cuda.synchronize()
    for b in range(2):
        sl = slice(b * seq, (b + 1) * seq)
        want = orc.flash_attention(q[sl].copy(), k[sl].copy(), v[sl].copy(), hd, scale=scale)
        assert np.max(np.abs(host(out)[sl] - want)) < 1e-4


@pytest.mark.parametrize("attn_len,heads,hd", [(1, 2, 4), (5, 3, 16), (33, 12, 64), (64, 12, 64)])
def test_cached_attention_three_dispatch(ak, orc, golden, torch_cuda, attn_len, heads, hd):
    torch = torch_cuda
    dim, max_ctx = heads * hd, 64
    q = orc.lcg(dim, 1)
    k = orc.lcg(max_ctx * dim, 2).reshape(max_ctx, dim)
    v = orc.lcg(max_ctx * dim, 3).reshape(max_ctx, dim)
    scores = nan_like(torch, heads * max_ctx)
    out = nan_like(torch, dim)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    dq, dk, dv = dev(torch, q), dev(torch, k), dev(torch, v)
    ak.ops.attn_qk_cached(dq, dk, scores, attn_len, dim, hd)
    ak.ops.softmax_rect(scores, heads, attn_len, scale)
    ak.ops.attn_av_cached(scores, dv, out, attn_len, dim, hd)
    torch.cuda.synchronize()
    want = orc.decode_attention(q, k, v, attn_len, hd)
    assert np.max(np.abs(host(out) - want)) < 1e-5
    key = f"cached_{attn_len}_{heads}_{hd}"
    if key in golden.files:
        assert np.max(np.abs(host(out) - golden[key])) < 1e-4
    # the meta bounds the live work: nothing past heads*attn_len was written
    assert np.isnan(host(scores)[heads * attn_len:]).all()


def test_gemv_routing(ak, orc, golden, torch_cuda):
    torch = torch_cuda
    n, k = 301, 19
    a, b, c0 = orc.lcg(k, 10), orc.lcg(k * n, 20).reshape(k, n), orc.lcg(n, 30)
    c = nan_like(torch, n)
    c_add = dev(torch, c0)
    ak.ops.matmul(dev(torch, a), dev(torch, b), c, 1, n, k)
    ak.ops.matmul_add(dev(torch, a), dev(torch, b), c_add, 1, n, k)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(c) - golden["gemv"])) < 1e-4
    assert np.max(np.abs(host(c_add) - golden["gemv_add"])) < 1e-4


@pytest.mark.parametrize("m,n,k", [(1, 2304, 768), (1, 768, 3072), (1, 50257, 768), (1, 7, 5), (2, 301, 19),
                                   (37, 130, 70), (64, 768, 768), (130, 2304, 96), (5, 3, 1)])
def test_matmul_and_matmul_add(ak, orc, torch_cuda, m, n, k):
    torch = torch_cuda
    a = orc.lcg(m * k, 1).reshape(m, k)
    b = (orc.lcg(k * n, 2) * np.float32(0.1)).reshape(k, n)
    c0 = orc.lcg(m * n, 3).reshape(m, n)
    c = nan_like(torch, m, n)
    c_add = dev(torch, c0)
    ak.ops.matmul(dev(torch, a), dev(torch, b), c, m, n, k)
    ak.ops.matmul_add(dev(torch, a), dev(torch, b), c_add, m, n, k)
    torch.cuda.synchronize()
    want = orc.matmul(a, b)
    tol = 2e-5 * max(1.0, np.sqrt(k))
    assert np.max(np.abs(host(c) - want)) < tol
    assert np.max(np.abs(host(c_add) - orc.matmul(a, b, c0))) < tol


def test_gemv_is_deterministic(ak, orc, torch_cuda):
    torch = torch_cuda
    n, k = 2304, 768
    a, b = dev(torch, orc.lcg(k, 4)), dev(torch, orc.lcg(k * n, 5))
    outs = []
    for _ in range(3):
        c = nan_like(torch, n)
        ak.ops.matmul(a, b, c, 1, n, k)
        torch.cuda.synchronize()
        outs.append(host(c))
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


def test_elementwise_ops_past_1d_grid_limit(ak, golden, torch_cuda):
    """src/nn/ops/emit.rs:1468-1504: 17,000,003 elements, probes around 65535*256."""
    torch = torch_cuda
    LEN = 17_000_003
    i = torch.arange(LEN, device="cuda", dtype=torch.int64)
    data = ((i % 1000).float() - 500.0) / 250.0
    res = (i % 777).float() / 777.0
    ak.ops.silu(data, LEN)
    torch.cuda.synchronize()
    got = host((data + res)[torch.from_numpy(golden["silu_probe_idx"]).cuda()])
    assert np.max(np.abs(got - golden["silu_probe_expected"])) < 1e-5


@pytest.mark.parametrize("rows,size", [(1, 768), (5, 24), (64, 768), (3, 2048), (7, 4100), (4, 19)])
def test_rmsnorm(ak, orc, torch_cuda, rows, size):
    torch = torch_cuda
    x = orc.lcg(rows * size, 7).reshape(rows, size)
    w = orc.lcg(size, 8)
    y = nan_like(torch, rows, size)
    ak.ops.rmsnorm(dev(torch, x), dev(torch, w), y, rows, size, 1e-5)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(y) - orc.rmsnorm(x, w, 1e-5))) < 2e-6 * max(1.0, float(np.abs(x).max() * 100))


def test_embedding_and_invalid_ids(ak, orc, torch_cuda):
    torch = torch_cuda
    table = orc.lcg(11 * 6, 9).reshape(11, 6)
    toks = np.array([3, 10, 11, 4000000000, 0], np.uint32)
    out = nan_like(torch, 5, 6)
    ak.ops.embedding(torch.from_numpy(toks.view(np.int32)).cuda(), dev(torch, table), out, 11, 6, 5)
    torch.cuda.synchronize()
    assert np.array_equal(host(out), orc.embedding(toks, table))


@pytest.mark.parametrize("seq,dim,hd,pos", [(8, 8, 4, 0), (37, 12, 4, 0), (65, 48, 16, 0), (1, 768, 64, 511), (3, 128, 128, 1000)])
def test_rope_and_rope_offset(ak, orc, torch_cuda, seq, dim, hd, pos):
    torch = torch_cuda
    x = orc.lcg(seq * dim, 10).reshape(seq, dim)
    d = dev(torch, x)
    if pos == 0:
        ak.ops.rope(d, seq, dim, hd)
    else:
        ak.ops.rope_offset(d, seq, dim, hd, pos)
    torch.cuda.synchronize()
    want = orc.rope(x, hd, pos)
    # angles reach ~1000 rad: one ulp of the angle is ~6e-5
    assert np.max(np.abs(host(d) - want)) < 1e-4
    if pos == 0 and seq <= 8:
        assert np.max(np.abs(host(d) - want)) < 2e-6


def test_head_gather_qkv_split_and_cache_write(ak, orc, torch_cuda):
    torch = torch_cuda
    seq, dim = 37, 12
    qkv = orc.lcg(seq * 3 * dim, 50).reshape(seq, 3 * dim)
    dq = dev(torch, qkv)
    parts = []
    for i in range(3):  # HeadMoveMeta::qkv_slice (src/nn/ops/meta.rs:52-59)
        dst = nan_like(torch, seq, dim)
        ak.ops.head_gather(dq, dst, seq, 3 * dim, dim, i * dim)
        parts.append(dst)
    torch.cuda.synchronize()
    for i in range(3):
        assert np.array_equal(host(parts[i]), qkv[:, i * dim:(i + 1) * dim])
    # last-row extraction (src/nn/inference.rs:125-135)
    last = nan_like(torch, dim)
    ak.ops.head_gather(parts[0], last, 1, dim, dim, (seq - 1) * dim)
    cache = torch.zeros(64, dim, device="cuda")
    ak.ops.cache_write(parts[1], cache, seq, dim, 5)
    torch.cuda.synchronize()
    assert np.array_equal(host(last), qkv[-1, :dim])
    c = host(cache)
    assert np.array_equal(c[5:5 + seq], qkv[:, dim:2 * dim]) and not c[:5].any() and not c[5 + seq:].any()


def test_argmax_first_max_and_kat(ak, golden, torch_cuda):
    torch = torch_cuda
    V = 50257
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((6, V)).astype(np.float32)
    logits[1, 40000] = logits[1, 123] = 9.0     # tie: lowest index wins (src/nn/sampling.rs:85-88)
    logits[2, :] = -3.0                          # all equal -> 0
    logits[3, V - 1] = 50.0
    logits[4, 0] = 50.0
    out = torch.full((6,), 77, dtype=torch.int32, device="cuda")
    ak.ops.argmax(dev(torch, logits), 6, V, out)
    kat = torch.full((1,), 77, dtype=torch.int32, device="cuda")
    ak.ops.argmax(dev(torch, golden["kat_logits"]), 1, 5, kat)
    torch.cuda.synchronize()
    want = [int(np.argmax(logits[i])) for i in range(6)]
    assert host(out).tolist() == want and want[1] == 123 and want[2] == 0
    assert host(kat).tolist() == [3]


@pytest.mark.parametrize("out_dtype", [0, 1])
@pytest.mark.parametrize("with_res,hd", [(False, 0), (True, 0), (True, 64), (False, 128)])
def test_rmsnorm_rope_residual_fused_vs_unfused(ak, orc, torch_cuda, out_dtype, with_res, hd):
    """The fused kernel equals the composition of the reference's unfused ops
    (the pattern of src/nn/ops/emit.rs:1101-1303)."""
    torch = torch_cuda
    rows, size = 70, 768
    x = orc.lcg(rows * size, 21).reshape(rows, size)
    r = orc.lcg(rows * size, 22).reshape(rows, size)
    w = (orc.lcg(size, 23) * np.float32(0.1) + np.float32(1.0)).astype(np.float32)
    pos = (np.arange(rows) * 7 % 300).astype(np.int32)
    dx = dev(torch, x)
    y = torch.full((rows, size), float("nan"), device="cuda", dtype=torch.float32 if out_dtype == 0 else torch.bfloat16)
    ak.ops.rmsnorm_rope_residual(dx, dev(torch, r) if with_res else None, dev(torch, w), y,
                                 torch.from_numpy(pos).cuda() if hd else None, rows, size, 1e-5, hd, out_dtype)
    torch.cuda.synchronize()
    h = (x + r).astype(np.float32) if with_res else x
    want = orc.rmsnorm(h, w, 1e-5)
    if hd:
        want = np.stack([orc.rope(want[i:i + 1], hd, int(pos[i]))[0] for i in range(rows)])
    got = host(y.float())
    tol = 2e-4 if out_dtype == 0 else 3e-2
    assert np.max(np.abs(got - want)) < tol
    if with_res:
        assert np.array_equal(host(dx), h)  # the residual stream is written back
