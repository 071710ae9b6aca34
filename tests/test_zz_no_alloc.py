"""GPU: the allocation-free decode attention entry point (`ak_attn_decode_paged_noalloc`).

It exists for hosts that may not allocate device memory at call time: a plugin inside another
framework's memory pool, a serving loop that forbids allocator calls once it is running, or a
process that has already given all free HBM to its KV pool. Its split-KV partials live in a
buffer inside the library image. This file checks, through the C ABI, that it returns what the
ordinary entry point (caller-provided scratch) returns and what the CPU oracle computes, on two
calls in a row that reuse the shared buffer, and that an over-sized request is refused instead
of overrunning the buffer.

Collected last on purpose (file name): a failure here cannot hide any other test's result.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(torch, ak, rows, heads, hd, max_len, seed, dtype):
    tdt = torch.bfloat16 if dtype == ak.AK_BF16 else torch.float32
    max_blocks = (max_len + 15) // 16
    n_blocks = rows * max_blocks + 5
    g = torch.Generator(device="cuda").manual_seed(seed)
    kp = torch.randn(n_blocks, heads, 16, hd, device="cuda", generator=g).to(tdt)
    vp = torch.randn(n_blocks, heads, 16, hd, device="cuda", generator=g).to(tdt)
    tables = torch.randperm(n_blocks, device="cuda", generator=g)[:rows * max_blocks].to(torch.int32).reshape(rows, max_blocks)
    q = torch.randn(rows, heads * hd, device="cuda", generator=g).to(tdt)
    lens = ak.uniform_ints(rows, 1, max_len, seed=seed).astype(np.int32)
    lens[0] = max_len
    return kp, vp, tables.contiguous(), q, torch.from_numpy(lens).cuda(), n_blocks, max_blocks


def _oracle_rows(orc, kp, vp, tables, q, kv_lens, heads, hd, rows):
    """The oracle's cached attention (src/shaders/cpu.rs:144-203) for a few rows, from the paged pools."""
    kp, vp, q = kp.float().cpu().numpy(), vp.float().cpu().numpy(), q.float().cpu().numpy()
    tables, kv_lens = tables.cpu().numpy(), kv_lens.cpu().numpy()
    out = {}
    for r in rows:
        L = int(kv_lens[r])
        pos = np.arange(L)
        k = kp[tables[r, pos // 16], :, pos % 16, :].reshape(L, heads * hd)
        v = vp[tables[r, pos // 16], :, pos % 16, :].reshape(L, heads * hd)
        out[r] = orc.decode_attention(q[r].copy(), np.ascontiguousarray(k), np.ascontiguousarray(v), L, hd)
    return out


@pytest.mark.parametrize("dtype_name", ["bf16", "f32"])
def test_noalloc_matches_scratch_entry_point_twice(ak, orc, torch_cuda, dtype_name):
    torch = torch_cuda
    dtype = ak.AK_BF16 if dtype_name == "bf16" else ak.AK_F32
    tol = 1e-2 if dtype == ak.AK_BF16 else 2e-5      # the tolerances of test_attn_decode_paged
    heads, hd, n_splits = 12, 64, 3
    assert ak.ops.attn_decode_noalloc_max_scratch_bytes() == 8 << 20
    # two different problems back to back: the second call finds the first call's partials in the buffer
    for call, (rows, max_len, seed) in enumerate([(20, 512, 11), (7, 300, 12)]):
        kp, vp, tables, q, kv_lens, n_blocks, max_blocks = _case(torch, ak, rows, heads, hd, max_len, seed, dtype)
        nbytes = ak.ops.attn_decode_scratch_bytes(rows, heads, hd, max_blocks, n_splits, dtype)
        assert 0 < nbytes <= ak.ops.attn_decode_noalloc_max_scratch_bytes()
        scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        want = torch.full_like(q, float("nan"))
        got = torch.full_like(q, float("nan"))
        ak.ops.attn_decode_paged(q, kp, vp, tables, kv_lens, want, rows, heads, hd, max_blocks, 0.125, dtype,
                                 n_splits, n_blocks, scratch)
        ak.ops.attn_decode_paged_noalloc(q, kp, vp, tables, kv_lens, got, rows, heads, hd, max_blocks, 0.125, dtype,
                                         n_splits, n_blocks)
        torch.cuda.synchronize()
        w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.isfinite(g).all(), f"call {call}: non-finite output"
        assert np.max(np.abs(g - w)) <= tol, f"call {call}: differs from the scratch entry point"
        # and against the CPU oracle directly (rows 0 = the longest sequence, 1 and the last one); values ~N(0,1),
        # so the bf16 bound is the output's rounding step at |x| < 4
        for r, want_row in _oracle_rows(orc, kp, vp, tables, q, kv_lens, heads, hd, (0, 1, rows - 1)).items():
            assert np.max(np.abs(g[r] - want_row)) <= (3e-2 if dtype == ak.AK_BF16 else 1e-4), f"call {call}, row {r}: differs from the oracle"


def test_noalloc_rejects_oversized_request(ak, torch_cuda):
    torch = torch_cuda
    rows, heads, hd, n_splits = 4096, 12, 64, 8       # 4096*12*8*66*4 B = 104 MB of partials > 8 MiB
    dummy = torch.zeros(16, device="cuda", dtype=torch.bfloat16)
    idx = torch.zeros(16, device="cuda", dtype=torch.int32)
    with pytest.raises(ak.AkashaError) as e:
        ak.ops.attn_decode_paged_noalloc(dummy, dummy, dummy, idx, idx, dummy, rows, heads, hd, 32, 0.125, ak.AK_BF16,
                                         n_splits, 0)
    assert e.value.kind == "Unsupported" and "exceed" in str(e.value)
    torch.cuda.synchronize()   # nothing was launched, the context is intact
