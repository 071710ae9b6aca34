"""ctypes front end of the CPU oracle (`akasha_oracle.c`).

Test infrastructure only: the test-suite, the smoke check and the benchmark's CPU-baseline leg
load this module to CHECK the CUDA library; the library itself never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libakasha_oracle.so")

u32p = C.POINTER(C.c_uint32)
f32p = C.POINTER(C.c_float)


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (see the Makefile beside this file)."""
    src = os.path.join(_HERE, "akasha_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.check_call(["make", "-C", _HERE, "-B", "libakasha_oracle.so"], env=env,
                              stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        L = _lib
        L.or_max_threads.restype = C.c_int
        L.or_set_threads.argtypes = [C.c_int]
        L.or_lcg_fill.argtypes = [f32p, C.c_uint64, C.c_uint64]
        L.or_round_bf16.argtypes = [f32p, C.c_uint64]
        L.or_embedding.argtypes = [u32p, f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32]
        L.or_rmsnorm.argtypes = [f32p, f32p, f32p, C.c_uint32, C.c_uint32, C.c_float]
        L.or_matmul.argtypes = [f32p, f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]
        L.or_head_gather.argtypes = [f32p, f32p] + [C.c_uint32] * 4
        L.or_rope.argtypes = [f32p] + [C.c_uint32] * 4
        L.or_cache_write.argtypes = [f32p, f32p] + [C.c_uint32] * 3
        L.or_attn_qk_cached.argtypes = [f32p, f32p, f32p] + [C.c_uint32] * 3
        L.or_softmax_rect.argtypes = [f32p, C.c_uint32, C.c_uint32, C.c_float]
        L.or_attn_av_cached.argtypes = [f32p, f32p, f32p] + [C.c_uint32] * 3
        L.or_silu.argtypes = [f32p, C.c_uint64]
        L.or_flash_attention.argtypes = [f32p, f32p, f32p, f32p, f32p, C.c_uint32, C.c_uint32,
                                         C.c_uint32, C.c_float, C.c_uint32]
        L.or_argmax.argtypes = [f32p, C.c_uint32]
        L.or_argmax.restype = C.c_uint32
        L.or_sample_greedy.argtypes = [f32p, C.c_uint32, u32p, C.c_uint32, C.c_float]
        L.or_sample_greedy.restype = C.c_uint32
        L.or_sample_token.argtypes = [f32p, C.c_uint32, C.c_float, C.c_uint32, C.c_float, u32p, C.c_uint32, C.c_float, C.c_double]
        L.or_sample_token.restype = C.c_uint32
        L.or_model_create.argtypes = [C.c_uint32] * 5 + [C.c_float, C.POINTER(f32p), C.c_int]
        L.or_model_create.restype = C.c_void_p
        L.or_model_destroy.argtypes = [C.c_void_p]
        L.or_session_create.argtypes = [C.c_void_p, C.c_uint32]
        L.or_session_create.restype = C.c_void_p
        L.or_session_destroy.argtypes = [C.c_void_p]
        L.or_session_reset.argtypes = [C.c_void_p]
        L.or_session_len.argtypes = [C.c_void_p]
        L.or_session_len.restype = C.c_uint32
        L.or_session_k.argtypes = [C.c_void_p, C.c_uint32]
        L.or_session_k.restype = f32p
        L.or_session_v.argtypes = [C.c_void_p, C.c_uint32]
        L.or_session_v.restype = f32p
        L.or_prefill.argtypes = [C.c_void_p, u32p, C.c_uint32, f32p]
        L.or_decode_step.argtypes = [C.c_void_p, C.c_uint32, f32p]
        L.or_generate_greedy.argtypes = [C.c_void_p, u32p, C.c_uint32, C.c_uint32, u32p, f32p,
                                         C.POINTER(C.c_int)]
        L.or_pool_create.argtypes = [C.c_uint32]
        L.or_pool_create.restype = C.c_void_p
        L.or_pool_destroy.argtypes = [C.c_void_p]
        L.or_pool_alloc.argtypes = [C.c_void_p]
        L.or_pool_alloc.restype = C.c_int64
        L.or_pool_free.argtypes = [C.c_void_p, C.c_uint32]
    return _lib


def _f(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(f32p)


def _u(a: np.ndarray):
    assert a.dtype == np.uint32 and a.flags.c_contiguous
    return a.ctypes.data_as(u32p)


def max_threads() -> int:
    return lib().or_max_threads()


def set_threads(n: int) -> None:
    lib().or_set_threads(n)


def lcg(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().or_lcg_fill(_f(out), n, seed)
    return out


def round_bf16(x: np.ndarray) -> np.ndarray:
    y = np.ascontiguousarray(x, np.float32).copy()
    lib().or_round_bf16(_f(y), y.size)
    return y


def embedding(tokens, table):
    tokens = np.ascontiguousarray(tokens, np.uint32)
    vocab, dim = table.shape
    out = np.full((tokens.size, dim), np.nan, np.float32)
    lib().or_embedding(_u(tokens), _f(table), _f(out), vocab, dim, tokens.size)
    return out


def rmsnorm(x, w, eps=1e-5):
    x2 = np.ascontiguousarray(x, np.float32).reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    lib().or_rmsnorm(_f(x2), _f(w), _f(out), x2.shape[0], x2.shape[1], eps)
    return out.reshape(x.shape)


def matmul(a, b, c=None):
    """c = a @ b, or c += a @ b when c is given (returns a new array)."""
    a2 = np.ascontiguousarray(a, np.float32).reshape(-1, a.shape[-1])
    m, k = a2.shape
    k2, n = b.shape
    assert k == k2
    if c is None:
        out = np.empty((m, n), np.float32)
        lib().or_matmul(_f(a2), _f(b), _f(out), m, n, k, 0)
    else:
        out = np.ascontiguousarray(c, np.float32).reshape(m, n).copy()
        lib().or_matmul(_f(a2), _f(b), _f(out), m, n, k, 1)
    return out


def head_gather(src, seq_len, full_dim, head_dim, head_offset):
    dst = np.empty((seq_len, head_dim), np.float32)
    lib().or_head_gather(_f(src), _f(dst), seq_len, full_dim, head_dim, head_offset)
    return dst


def rope(x, head_dim, pos_offset=0):
    y = np.ascontiguousarray(x, np.float32).reshape(-1, x.shape[-1]).copy()
    lib().or_rope(_f(y), y.shape[0], y.shape[1], head_dim, pos_offset)
    return y.reshape(x.shape)


def cache_write(src, cache, dst_row_offset):
    src2 = np.ascontiguousarray(src, np.float32).reshape(-1, cache.shape[1])
    lib().or_cache_write(_f(src2), _f(cache), src2.shape[0], cache.shape[1], dst_row_offset)


def attn_qk_cached(q, k_cache, attn_len, head_dim):
    dim = q.size
    scores = np.empty((dim // head_dim, attn_len), np.float32)
    lib().or_attn_qk_cached(_f(q), _f(k_cache), _f(scores), attn_len, dim, head_dim)
    return scores


def softmax_rect(scores, scale):
    y = np.ascontiguousarray(scores, np.float32).copy()
    lib().or_softmax_rect(_f(y), y.shape[0], y.shape[1], scale)
    return y


def attn_av_cached(probs, v_cache, head_dim):
    heads, attn_len = probs.shape
    dim = heads * head_dim
    out = np.empty(dim, np.float32)
    lib().or_attn_av_cached(_f(probs), _f(v_cache), _f(out), attn_len, dim, head_dim)
    return out


def decode_attention(q, k_cache, v_cache, attn_len, head_dim):
    """The reference's three-dispatch decode attention (qk -> softmax_rect -> av)."""
    s = attn_qk_cached(q, k_cache, attn_len, head_dim)
    p = softmax_rect(s, 1.0 / np.sqrt(np.float32(head_dim)))
    return attn_av_cached(p, v_cache, head_dim)


def silu(x):
    y = np.ascontiguousarray(x, np.float32).copy()
    lib().or_silu(_f(y), y.size)
    return y


def flash_attention(q, k, v, head_dim, scale=None, with_lse=False):
    seq, dim = q.shape
    if scale is None:
        scale = float(np.float32(1.0) / np.sqrt(np.float32(head_dim)))
    out = np.empty((seq, dim), np.float32)
    lse = np.empty((seq, dim // head_dim), np.float32)
    lib().or_flash_attention(_f(q), _f(k), _f(v), _f(out), _f(lse), seq, dim, head_dim, scale, 0)
    return (out, lse) if with_lse else out


def argmax(logits) -> int:
    logits = np.ascontiguousarray(logits, np.float32)
    return int(lib().or_argmax(_f(logits), logits.size))


def sample_greedy(logits, seen=(), penalty=1.0) -> int:
    logits = np.ascontiguousarray(logits, np.float32)
    seen = np.ascontiguousarray(seen, np.uint32)
    return int(lib().or_sample_greedy(_f(logits), logits.size, _u(seen), seen.size, penalty))


def sample_token(logits, temperature, top_k, top_p, seen=(), penalty=1.0, r=0.5) -> int:
    """`sample_token` (src/nn/sampling.rs:18-81) with the uniform draw r supplied."""
    logits = np.ascontiguousarray(logits, np.float32)
    seen = np.ascontiguousarray(seen, np.uint32)
    return int(lib().or_sample_token(_f(logits), logits.size, temperature, top_k, top_p, _u(seen), seen.size, penalty, r))


class Model:
    """Borrowed-weight model: `params` is the list of arrays in `ModelWeights::params()` order."""

    def __init__(self, cfg, params, act_bf16=False):
        self.cfg = cfg
        self.params = [np.ascontiguousarray(p, np.float32) for p in params]
        assert len(self.params) == 3 + 6 * cfg["num_layers"]
        arr = (f32p * len(self.params))(*[_f(p) for p in self.params])
        self._arr = arr
        self.h = lib().or_model_create(cfg["vocab_size"], cfg["dim"], cfg["num_heads"],
                                       cfg["num_layers"], cfg["ffn_hidden"], cfg["norm_eps"], arr,
                                       int(act_bf16))

    def __del__(self):
        if getattr(self, "h", None):
            lib().or_model_destroy(self.h)
            self.h = None


class Session:
    def __init__(self, model: Model, max_ctx: int):
        self.model = model
        self.max_ctx = max_ctx
        self.h = lib().or_session_create(model.h, max_ctx)

    def __del__(self):
        if getattr(self, "h", None):
            lib().or_session_destroy(self.h)
            self.h = None

    def reset(self):
        lib().or_session_reset(self.h)

    @property
    def cur_len(self):
        return lib().or_session_len(self.h)

    def prefill(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.uint32)
        logits = np.empty(self.model.cfg["vocab_size"], np.float32)
        rc = lib().or_prefill(self.h, _u(tokens), tokens.size, _f(logits))
        return rc, logits

    def decode_step(self, token):
        logits = np.empty(self.model.cfg["vocab_size"], np.float32)
        rc = lib().or_decode_step(self.h, int(token), _f(logits))
        return rc, logits

    def generate_greedy(self, prompt, steps, want_logits=False):
        prompt = np.ascontiguousarray(prompt, np.uint32)
        toks = np.zeros(steps, np.uint32)
        V = self.model.cfg["vocab_size"]
        logits = np.empty((steps + 1, V), np.float32) if want_logits else None
        st = C.c_int(0)
        n = lib().or_generate_greedy(self.h, _u(prompt), prompt.size, steps, _u(toks),
                                     _f(logits) if want_logits else None, C.byref(st))
        return st.value, toks[:n], logits

    def cache(self, layer):
        D = self.model.cfg["dim"]
        n = self.cur_len
        k = np.ctypeslib.as_array(lib().or_session_k(self.h, layer), (self.max_ctx, D))[:n].copy()
        v = np.ctypeslib.as_array(lib().or_session_v(self.h, layer), (self.max_ctx, D))[:n].copy()
        return k, v


class BlockPool:
    """Lowest-free-index-first block allocator (the engine's slot rule)."""

    def __init__(self, n_blocks):
        self.h = lib().or_pool_create(n_blocks)

    def alloc(self) -> int:
        return int(lib().or_pool_alloc(self.h))

    def free(self, b: int):
        lib().or_pool_free(self.h, b)

    def __del__(self):
        if getattr(self, "h", None):
            lib().or_pool_destroy(self.h)
            self.h = None
