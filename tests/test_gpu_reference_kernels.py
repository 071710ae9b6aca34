"""GPU: this library's kernels against the REFERENCE'S OWN CUDA kernels on the same B200, same inputs.

`oracle/make_ref.py` compiles the kernel strings of the reference's src/shaders/cuda.rs, unchanged,
with nvcc into `oracle/_ref/libakasha_refkernels_cuda.so` (built where the reference sources are
present; the built file travels with the repository to the GPU box, the sources do not). Each
test launches a reference kernel with the grid its emitter uses (src/nn/ops/emit.rs) and the
matching entry point of this library on the same device buffers, and compares the results.
Skipped when that library has not been built.
"""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libakasha_refkernels_cuda.so")


@pytest.fixture(scope="module")
def ref(torch_cuda):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libakasha_refkernels_cuda.so not built (python oracle/make_ref.py)")
    return C.CDLL(REF_SO)


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def meta(torch, *vals):
    out = np.zeros(len(vals), np.uint32)
    for i, v in enumerate(vals):
        out[i] = np.float32(v).view(np.uint32) if isinstance(v, float) else np.uint32(v)
    return torch.from_numpy(out.view(np.int32)).cuda()


def launch(ref, entry, grid, *bufs):
    fn = getattr(ref, "ref_cuda_" + entry)
    fn.restype = C.c_int
    args = [C.c_void_p(0), C.c_uint(grid[0]), C.c_uint(grid[1]), C.c_uint(grid[2])]
    for b in bufs:
        args.append(C.c_void_p(b.data_ptr()) if hasattr(b, "data_ptr") else b)
    rc = fn(*args)
    assert rc == 0, f"{entry}: launch failed with CUDA error {rc}"


def host(t):
    return t.detach().float().cpu().numpy()


def test_embedding_rmsnorm_silu(ak, orc, ref, torch_cuda):
    torch = torch_cuda
    vocab, dim = 5003, 768
    table = dev(torch, orc.lcg(vocab * dim, 40).reshape(vocab, dim))
    toks = torch.from_numpy(np.array([3, 41, 7, vocab - 1, 0, 25, vocab, 2_000_000_000], np.int64).astype(np.int32)).cuda()
    seq = toks.numel()
    want = torch.full((seq, dim), float("nan"), device="cuda")
    got = torch.full((seq, dim), float("nan"), device="cuda")
    launch(ref, "embedding_kernel", ((dim + 255) // 256, seq, 1), toks, table, want, meta(torch, vocab, dim, seq))
    ak.ops.embedding(toks, table, got, vocab, dim, seq)
    torch.cuda.synchronize()
    assert np.array_equal(host(got), host(want))            # a copy: bit-exact, out-of-range ids give zeros

    for rows, size in ((5, 32), (64, 768), (2, 1000)):
        x = dev(torch, orc.lcg(rows * size, 80).reshape(rows, size) * 3.0)
        w = dev(torch, 1.0 + 0.1 * orc.lcg(size, 81))
        want = torch.full((rows, size), float("nan"), device="cuda")
        got = torch.full((rows, size), float("nan"), device="cuda")
        launch(ref, "rmsnorm_kernel", (rows, 1, 1), x, w, want, meta(torch, rows, size, 1e-5))
        ak.ops.rmsnorm(x, w, got, rows, size, 1e-5)
        torch.cuda.synchronize()
        assert np.max(np.abs(host(got) - host(want))) < 1e-5  # summation order differs (tree vs warp shuffle)

    n = 100_003
    x0 = orc.lcg(n, 60) * 6.0
    a, b = dev(torch, x0), dev(torch, x0)
    total = (n + 255) // 256
    gx = min(max(total, 1), 8192)
    launch(ref, "silu_kernel", (gx, (total + gx - 1) // gx, 1), a, C.c_uint(n))
    ak.ops.silu(b, n)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(a) - host(b))) < 1e-6


@pytest.mark.parametrize("seq,dim,hd", [(8, 8, 4), (37, 12, 4), (65, 48, 16), (16, 768, 64)])
def test_rope_and_rope_offset(ak, orc, ref, torch_cuda, seq, dim, hd):
    torch = torch_cuda
    x0 = orc.lcg(seq * dim, 10).reshape(seq, dim)
    a, b = dev(torch, x0), dev(torch, x0)
    launch(ref, "rope_kernel", ((hd // 2 + 15) // 16, (seq + 15) // 16, dim // hd), a, meta(torch, seq, dim, hd))
    ak.ops.rope(b, seq, dim, hd)
    torch.cuda.synchronize()
    # the reference kernel uses the device's float powf/cosf/sinf, this library rounds double-precision results once
    assert np.max(np.abs(host(a) - host(b))) < 2e-5
    for pos in (7, 300, 511):
        y0 = orc.lcg(dim, 20).reshape(1, dim)
        a, b = dev(torch, y0), dev(torch, y0)
        launch(ref, "rope_offset_kernel", ((hd // 2 + 15) // 16, 1, dim // hd), a, meta(torch, 1, dim, hd, pos))
        ak.ops.rope_offset(b, 1, dim, hd, pos)
        torch.cuda.synchronize()
        assert np.max(np.abs(host(a) - host(b))) < 1e-4   # |angle| up to 511 rad: float sin/cos argument reduction


def test_head_gather_and_cache_write(ak, orc, ref, torch_cuda):
    torch = torch_cuda
    seq, dim = 37, 768
    qkv = dev(torch, orc.lcg(seq * 3 * dim, 50).reshape(seq, 3 * dim))
    for part in range(3):
        want = torch.full((seq, dim), float("nan"), device="cuda")
        got = torch.full((seq, dim), float("nan"), device="cuda")
        launch(ref, "head_gather_kernel", ((dim + 15) // 16, (seq + 15) // 16, 1), qkv, want, meta(torch, seq, 3 * dim, dim, part * dim))
        ak.ops.head_gather(qkv, got, seq, 3 * dim, dim, part * dim)
        torch.cuda.synchronize()
        assert np.array_equal(host(got), host(want))
    cache0 = orc.lcg(64 * dim, 70).reshape(64, dim)
    src = dev(torch, orc.lcg(3 * dim, 71).reshape(3, dim))
    a, b = dev(torch, cache0), dev(torch, cache0)
    launch(ref, "cache_write_kernel", ((dim + 15) // 16, (3 + 15) // 16, 1), src, a, meta(torch, 3, dim, 5))
    ak.ops.cache_write(src, b, 3, dim, 5)
    torch.cuda.synchronize()
    assert np.array_equal(host(a), host(b))


@pytest.mark.parametrize("L,heads,hd", [(1, 2, 4), (5, 3, 16), (33, 12, 64), (300, 12, 64), (512, 12, 64)])
def test_cached_attention_chain_and_fused_decode_attention(ak, orc, ref, torch_cuda, L, heads, hd):
    """attn_qk_cached -> softmax_rect -> attn_av_cached of the reference (one sequence, contiguous cache), this
    library's three emitters, and the fused paged decode attention, on the same K/V."""
    torch = torch_cuda
    dim, cap = heads * hd, max(64, L)
    q = dev(torch, orc.lcg(dim, 1))
    kc_h, vc_h = orc.lcg(cap * dim, 2).reshape(cap, dim), orc.lcg(cap * dim, 3).reshape(cap, dim)
    kc, vc = dev(torch, kc_h), dev(torch, vc_h)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    m3 = meta(torch, L, dim, hd)
    s_ref = torch.full((heads, L), float("nan"), device="cuda")
    o_ref = torch.full((dim,), float("nan"), device="cuda")
    launch(ref, "attn_qk_cached_kernel", ((L + 255) // 256, heads, 1), q, kc, s_ref, m3)
    raw_scores = host(s_ref).copy()
    launch(ref, "softmax_rect_kernel", ((heads + 255) // 256, 1, 1), s_ref, meta(torch, heads, L, scale))
    launch(ref, "attn_av_cached_kernel", ((dim + 255) // 256, 1, 1), s_ref, vc, o_ref, m3)
    s_mine = torch.full((heads, L), float("nan"), device="cuda")
    o_mine = torch.full((dim,), float("nan"), device="cuda")
    ak.ops.attn_qk_cached(q, kc, s_mine, L, dim, hd)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(s_mine) - raw_scores)) < 1e-5
    ak.ops.softmax_rect(s_mine, heads, L, scale)
    ak.ops.attn_av_cached(s_mine, vc, o_mine, L, dim, hd)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(s_mine) - host(s_ref))) < 1e-6
    assert np.max(np.abs(host(o_mine) - host(o_ref))) < 1e-5
    # the fused kernel reads the same rows from a paged pool [blocks, heads, 16, hd] through an identity table
    nb = (cap + 15) // 16
    pad = np.zeros((nb * 16, dim), np.float32)
    pad[:cap] = kc_h
    kp = dev(torch, pad.reshape(nb, 16, heads, hd).transpose(0, 2, 1, 3))
    pad[:cap] = vc_h
    vp = dev(torch, pad.reshape(nb, 16, heads, hd).transpose(0, 2, 1, 3))
    table = torch.arange(nb, dtype=torch.int32, device="cuda").reshape(1, nb)
    kv_len = torch.tensor([L], dtype=torch.int32, device="cuda")
    o_fused = torch.full((1, dim), float("nan"), device="cuda")
    ak.ops.attn_decode_paged(q.reshape(1, dim), kp, vp, table, kv_len, o_fused, 1, heads, hd, nb, scale, ak.AK_F32, 1, nb)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(o_fused)[0] - host(o_ref))) < 2e-5


@pytest.mark.parametrize("seq,heads,hd", [(8, 2, 4), (37, 3, 16), (65, 12, 64), (200, 12, 64)])
def test_flash_attention(ak, orc, ref, torch_cuda, seq, heads, hd):
    torch = torch_cuda
    dim = heads * hd
    q, k, v = (dev(torch, orc.lcg(seq * dim, s).reshape(seq, dim)) for s in (1, 2, 3))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    want = torch.full((seq, dim), float("nan"), device="cuda")
    lse_ref = torch.full((seq, heads), float("nan"), device="cuda")
    got = torch.full((seq, dim), float("nan"), device="cuda")
    lse = torch.full((seq, heads), float("nan"), device="cuda")
    launch(ref, "flash_attention_kernel", ((seq + 63) // 64, heads, 1), q, k, v, want, lse_ref, meta(torch, seq, dim, hd, scale, 0))
    ak.ops.flash_attention(q, k, v, got, seq, dim, hd, scale, 0, lse)
    torch.cuda.synchronize()
    assert np.max(np.abs(host(got) - host(want))) < 1e-5
    assert np.max(np.abs(host(lse) - host(lse_ref))) < 1e-4
