"""Generates `reference_test_math.npz`: known-answer vectors for the oracle.

The reference keeps no stored vectors; its tests compare kernels against plain Rust math written
inside the test modules. This script restates THAT in-test math in numpy float32 (independently
of `oracle/akasha_oracle.c`) on the reference's own shapes, seeds and input generator:

  * causal full-softmax attention      src/nn/ops/emit.rs:931-999, shapes 1002-1006, seeds 1015-1017
  * cached (decode) attention          src/nn/ops/emit.rs:1385-1411, shapes 1333-1337, max_ctx 64
  * GEMV / GEMV_ADD dot products       src/nn/ops/emit.rs:1449-1455, n=301, k=19, seeds 10/20/30
  * silu + residual at probe indices   src/nn/ops/emit.rs:1476-1501
  * greedy / repetition-penalty KATs   src/nn/sampling.rs:95-141
  * input generator (64-bit LCG)       src/nn/ops/emit.rs:910-921

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np

F = np.float32


def lcg(n, seed):
    """emit.rs:910-921"""
    mask = (1 << 64) - 1
    state = (seed + 0x9E3779B97F4A7C15) & mask
    out = np.empty(n, F)
    for i in range(n):
        state = (state * 6364136223846793005 + 1442695040888963407) & mask
        bits = (state >> 40) & 0x00FFFFFF
        out[i] = F(F(bits) / F(0x00FFFFFF)) * F(2.0) - F(1.0)
    return out


def seq_sum(x):
    """f32 left-to-right sum, like Rust's `.sum::<f32>()`."""
    acc = F(0.0)
    for v in x:
        acc = F(acc + v)
    return acc


def causal_attention(q, k, v, seq, dim, hd):
    """emit.rs:931-999 (forward part): per head, full softmax per row, causal."""
    scale = F(1.0) / np.sqrt(F(hd))
    out = np.zeros((seq, dim), F)
    for h0 in range(0, dim, hd):
        for i in range(seq):
            row = np.zeros(i + 1, F)
            for j in range(i + 1):
                row[j] = scale * seq_sum(q[i, h0:h0 + hd] * k[j, h0:h0 + hd])
            mx = row.max()
            row = np.exp(row - mx).astype(F)
            row = (row / seq_sum(row)).astype(F)
            for j in range(i + 1):
                out[i, h0:h0 + hd] = out[i, h0:h0 + hd] + row[j] * v[j, h0:h0 + hd]
    return out


def cached_attention(q, k, v, attn_len, heads, hd):
    """emit.rs:1385-1411"""
    d = heads * hd
    scale = F(1.0) / np.sqrt(F(hd))
    out = np.zeros(d, F)
    for h in range(heads):
        o = h * hd
        p = np.array([scale * seq_sum(q[o:o + hd] * k[j, o:o + hd]) for j in range(attn_len)], F)
        p = np.exp(p - p.max()).astype(F)
        s = seq_sum(p)
        for j in range(attn_len):
            pj = F(p[j] / s)
            out[o:o + hd] = out[o:o + hd] + pj * v[j, o:o + hd]
    return out


def main():
    g = {}
    for (seq, heads, hd) in [(8, 2, 4), (37, 3, 16), (65, 12, 64)]:
        dim = heads * hd
        n = seq * dim
        q, k, v = lcg(n, 1).reshape(seq, dim), lcg(n, 2).reshape(seq, dim), lcg(n, 3).reshape(seq, dim)
        g[f"flash_{seq}_{heads}_{hd}"] = causal_attention(q, k, v, seq, dim, hd)
    for (al, heads, hd) in [(1, 2, 4), (5, 3, 16), (33, 12, 64)]:
        dim, max_ctx = heads * hd, 64
        q = lcg(dim, 1)
        k = lcg(max_ctx * dim, 2).reshape(max_ctx, dim)
        v = lcg(max_ctx * dim, 3).reshape(max_ctx, dim)
        g[f"cached_{al}_{heads}_{hd}"] = cached_attention(q, k, v, al, heads, hd)
    n, kk = 301, 19
    a, b, c0 = lcg(kk, 10), lcg(kk * n, 20).reshape(kk, n), lcg(n, 30)
    dots = np.array([seq_sum(a * b[:, j]) for j in range(n)], F)
    g["gemv"] = dots
    g["gemv_add"] = (c0 + dots).astype(F)
    # elementwise probe (emit.rs:1476-1501)
    LEN, BOUNDARY = 17_000_003, 65535 * 256
    idx = np.array([0, BOUNDARY - 1, BOUNDARY, 16_900_000, LEN - 1], np.int64)
    data = ((idx % 1000).astype(F) - F(500.0)) / F(250.0)
    res = (idx % 777).astype(F) / F(777.0)
    g["silu_probe_idx"] = idx
    g["silu_probe_expected"] = (data / (F(1.0) + np.exp(-data).astype(F)) + res).astype(F)
    # sampling KATs (sampling.rs:95-141)
    g["kat_logits"] = np.array([1.0, 4.0, 2.0, 8.0, 3.0], F)
    g["kat_greedy"] = np.array([3], np.uint32)
    g["kat_penalty_seen"] = np.array([3], np.uint32)
    g["kat_penalty_value"] = np.array([100.0], F)
    g["kat_penalty_greedy"] = np.array([1], np.uint32)
    # generator spot values
    g["lcg_seed1_first8"] = lcg(8, 1)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_test_math.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, {k: v.shape for k, v in g.items()})


if __name__ == "__main__":
    main()
