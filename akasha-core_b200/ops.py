"""Emitter-level operators: one function per forward/cached emitter of the reference's
`src/nn/ops/emit.rs`, same names, same meta fields, running the sm_100a kernels through the C ABI.

Buffers are DEVICE memory: pass a raw pointer (int) or any object with `.data_ptr()` (a CUDA
torch tensor). Nothing here computes on the host. `stream` is a `cudaStream_t` as int (0/None =
default stream).
"""
from __future__ import annotations

import ctypes as C

from . import (AK_BF16, AK_F32, AttnCachedMeta, AttnDecodeParams, CacheWriteMeta, EmbeddingMeta, FlashAttnMeta,
               HeadMoveMeta, MatMulMeta, NormMeta, RopeMeta, RopeOffsetMeta, SoftmaxRectMeta, check, lib)


def _p(x):
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    return C.c_void_p(int(x))


def _s(stream):
    return C.c_void_p(int(stream)) if stream else None


def embedding(tokens, table, output, vocab_size, dim, seq_len, stream=None):  # emit.rs:228-257
    check(lib().ak_embedding(_s(stream), _p(tokens), _p(table), _p(output), EmbeddingMeta(vocab_size, dim, seq_len)))


def rmsnorm(input, weight, output, seq_len, size, eps=1e-5, stream=None):  # emit.rs:151-180
    check(lib().ak_rmsnorm(_s(stream), _p(input), _p(weight), _p(output), NormMeta(seq_len, size, eps)))


def matmul(a, b, c, m, n, k, stream=None):  # emit.rs:23-57 (m == 1 routes to the GEMV)
    check(lib().ak_matmul(_s(stream), _p(a), _p(b), _p(c), MatMulMeta(m, n, k)))


def matmul_add(a, b, c, m, n, k, stream=None):  # emit.rs:92-126
    check(lib().ak_matmul_add(_s(stream), _p(a), _p(b), _p(c), MatMulMeta(m, n, k)))


def head_gather(src, dst, seq_len, full_dim, head_dim, head_offset, stream=None):  # emit.rs:406-424
    check(lib().ak_head_gather(_s(stream), _p(src), _p(dst), HeadMoveMeta(seq_len, full_dim, head_dim, head_offset)))


def rope(vec, seq_len, dim, head_dim, row_offset=0, stream=None):  # emit.rs:306-313
    check(lib().ak_rope(_s(stream), _p(vec), RopeMeta(seq_len, dim, head_dim, row_offset)))


def rope_offset(vec, seq_len, dim, head_dim, pos, stream=None):  # emit.rs:325-342
    check(lib().ak_rope_offset(_s(stream), _p(vec), RopeOffsetMeta(seq_len, dim, head_dim, pos)))


def cache_write(src, cache, row_count, width, dst_row_offset, stream=None):  # emit.rs:649-675
    check(lib().ak_cache_write(_s(stream), _p(src), _p(cache), CacheWriteMeta(row_count, width, dst_row_offset)))


def attn_qk_cached(q, k_cache, scores, attn_len, dim, head_dim, stream=None):  # emit.rs:485-504
    check(lib().ak_attn_qk_cached(_s(stream), _p(q), _p(k_cache), _p(scores), AttnCachedMeta(attn_len, dim, head_dim)))


def softmax_rect(x, num_rows, width, scale, stream=None):  # emit.rs:528-542
    check(lib().ak_softmax_rect(_s(stream), _p(x), SoftmaxRectMeta(num_rows, width, scale)))


def attn_av_cached(scores, v_cache, out, attn_len, dim, head_dim, stream=None):  # emit.rs:507-525
    check(lib().ak_attn_av_cached(_s(stream), _p(scores), _p(v_cache), _p(out), AttnCachedMeta(attn_len, dim, head_dim)))


def flash_attention(q, k, v, out, seq_len, dim, head_dim, scale, row_offset=0, l_cache=None, stream=None):  # emit.rs:556-597
    check(lib().ak_flash_attention(_s(stream), _p(q), _p(k), _p(v), _p(out), _p(l_cache),
                                   FlashAttnMeta(seq_len, dim, head_dim, scale, row_offset)))


def silu(x, n, stream=None):  # emit.rs:686-696
    check(lib().ak_silu(_s(stream), _p(x), n))


def argmax(logits, rows, n, out_idx, stream=None):  # src/nn/sampling.rs:83-91 on the device
    check(lib().ak_argmax(_s(stream), _p(logits), rows, n, _p(out_idx)))


def sample_token(logits, rows, n, out_idx, temperature, top_k, top_p, seed, step, seen=None, seen_off=None,
                 repetition_penalty=1.0, stream=None):
    """`sample_token` (src/nn/sampling.rs:18-81) on the device; see the header for the RNG contract."""
    check(lib().ak_sample_token(_s(stream), _p(logits), rows, n, _p(seen), _p(seen_off), repetition_penalty, temperature,
                                top_k, top_p, seed, step, _p(out_idx)))


def sampler_uniform(seed: int, step: int, row: int) -> float:
    """The uniform number the device sampler draws for (seed, step, row)."""
    M = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)
    b = mix(seed ^ mix((step * 0x632BE59BD9B4E019 + row + 1) & M))
    return (b >> 11) / 9007199254740992.0


# ---- fused sm_100a kernels -----------------------------------------------------------------
def attn_decode_scratch_bytes(rows, heads, head_dim, max_blocks_per_seq, n_splits=0, kv_dtype=AK_BF16):
    p = AttnDecodeParams(rows, heads, head_dim, 16, max_blocks_per_seq, 0.0, kv_dtype, n_splits, 0)
    return int(lib().ak_attn_decode_scratch_bytes(C.byref(p)))


def attn_decode_paged(q, k_pool, v_pool, block_tables, kv_lens, out, rows, heads, head_dim, max_blocks_per_seq,
                      scale, kv_dtype=AK_BF16, n_splits=0, pool_blocks=0, scratch=None, stream=None):
    p = AttnDecodeParams(rows, heads, head_dim, 16, max_blocks_per_seq, scale, kv_dtype, n_splits, pool_blocks)
    check(lib().ak_attn_decode_paged(_s(stream), _p(q), _p(k_pool), _p(v_pool), _p(block_tables), _p(kv_lens),
                                     _p(out), _p(scratch), p))


def attn_decode_append_paged(qkv, rope_table, rope_len, k_pool, v_pool, block_tables, kv_lens, out, rows, heads, head_dim,
                             max_blocks_per_seq, scale, kv_dtype=AK_BF16, n_splits=0, pool_blocks=0, scratch=None, stream=None):
    """Decode attention with the new token's head split, RoPE and cache append fused in (`kv_lens`
    counts the new token; `rope_table` is float32 [rope_len, head_dim/2, 2] = (cos, sin))."""
    p = AttnDecodeParams(rows, heads, head_dim, 16, max_blocks_per_seq, scale, kv_dtype, n_splits, pool_blocks)
    check(lib().ak_attn_decode_append_paged(_s(stream), _p(qkv), _p(rope_table), rope_len, _p(k_pool), _p(v_pool),
                                            _p(block_tables), _p(kv_lens), _p(out), _p(scratch), p))


def attn_decode_paged_noalloc(q, k_pool, v_pool, block_tables, kv_lens, out, rows, heads, head_dim, max_blocks_per_seq,
                              scale, kv_dtype=AK_BF16, n_splits=0, pool_blocks=0, stream=None):
    """`attn_decode_paged` for callers that must not allocate: the split-KV partials live in a
    fixed buffer inside the library (8 MiB per GPU), no scratch argument, no cudaMalloc. Raises
    `Unsupported` when the partials would not fit. Calls that can overlap on one GPU share the
    buffer and must be ordered by the caller; make the first call on a device outside any capture."""
    p = AttnDecodeParams(rows, heads, head_dim, 16, max_blocks_per_seq, scale, kv_dtype, n_splits, pool_blocks)
    check(lib().ak_attn_decode_paged_noalloc(_s(stream), _p(q), _p(k_pool), _p(v_pool), _p(block_tables),
                                             _p(kv_lens), _p(out), p))


def attn_decode_noalloc_max_scratch_bytes() -> int:
    return int(lib().ak_attn_decode_noalloc_max_scratch_bytes())


def attn_prefill_paged(q, k_pool, v_pool, block_tables, max_blocks_per_seq, cu, seq_slot, out, n_seqs, max_len, q_rows,
                       heads, head_dim, scale, dtype=AK_BF16, pool_blocks=0, stream=None):
    """Causal attention of a ragged batch of newly prefilled sequences over the paged pools
    (the prefill graph's FLASH_ATTENTION node, src/nn/inference_graphs.rs:271-285)."""
    check(lib().ak_attn_prefill_paged(_s(stream), _p(q), _p(k_pool), _p(v_pool), _p(block_tables), max_blocks_per_seq, _p(cu),
                                      _p(seq_slot), _p(out), n_seqs, max_len, q_rows, heads, head_dim, scale, dtype,
                                      pool_blocks))


def rope_kv_append(qkv, positions, slots, q_out, k_pool, v_pool, tokens, heads, head_dim, kv_dtype=AK_BF16,
                   stream=None):
    check(lib().ak_rope_kv_append(_s(stream), _p(qkv), _p(positions), _p(slots), _p(q_out), _p(k_pool), _p(v_pool),
                                  tokens, heads, head_dim, 16, kv_dtype))


def rmsnorm_rope_residual(x, residual, weight, y, positions, rows, size, eps=1e-5, head_dim=0, out_dtype=AK_F32,
                          stream=None):
    check(lib().ak_rmsnorm_rope_residual(_s(stream), _p(x), _p(residual), _p(weight), _p(y), _p(positions), rows,
                                         size, eps, head_dim, out_dtype))


def gemm_bf16(a, wt, c, m, n, k, epilogue=0, stream=None, ldc=0):
    """C[m,n] (op)= A[m,k] @ Wt[n,k]^T on the tensor cores; `ldc` = row pitch of C in elements (0 = n)."""
    if ldc:
        check(lib().ak_gemm_bf16_ld(_s(stream), _p(a), _p(wt), _p(c), MatMulMeta(m, n, k), epilogue, ldc))
    else:
        check(lib().ak_gemm_bf16(_s(stream), _p(a), _p(wt), _p(c), MatMulMeta(m, n, k), epilogue))


def transpose_to_bf16(w_kn, wt_nk, k, n, stream=None):
    check(lib().ak_transpose_to_bf16(_s(stream), _p(w_kn), _p(wt_nk), k, n))
