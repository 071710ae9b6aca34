"""akasha-core_b200: host-side mirror of the akasha-core inference interface over the sm_100a C ABI.

The product is `libakasha_b200.so` (hand-written CUDA for B200, `include/akasha_b200.h`).
This module binds it with ctypes and mirrors the reference's names for the Prefill/Decode path:

* `ModelConfig`            -- src/config.rs:2-61
* `ModelWeights`           -- src/nn/weights.rs:40-47, tensors in `params()` order (158-171)
* `InferenceSession`       -- src/nn/inference.rs:13-327 (`prefill`, `decode_step`, `generate`,
                              `replace_cache`, `take_cache`)
* `ops.*`                  -- one function per emitter of src/nn/ops/emit.rs on the path
* `Engine`                 -- continuous batching (new; no counterpart in the reference)

There is NO CPU fallback: every compute call goes to the CUDA library and raises if the library
is missing or reports an error.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libakasha_b200.so")

AK_F32, AK_BF16 = 0, 1
EPI_STORE_F32, EPI_ADD_F32, EPI_STORE_BF16, EPI_SILU_BF16 = 0, 1, 2, 3


class AkashaError(RuntimeError):
    """Mirrors `AkashaError` (src/lib.rs:10-17); `code` is the C ABI status."""

    NAMES = {1: "EmptyPrompt", 2: "PromptTooLong", 3: "ContextFull", 4: "NoCache", 5: "CacheNotEmpty",
             100: "InvalidArg", 101: "Cuda", 102: "Alloc", 103: "Unsupported", 104: "DeviceWait",
             105: "NoCapacity", 106: "NotFound"}

    def __init__(self, code: int, msg: str):
        self.code = code
        self.kind = self.NAMES.get(code, f"Status{code}")
        super().__init__(f"{self.kind}: {msg}")


# ------------------------------------------------------------------ C structs
class _ModelConfig(C.Structure):
    _fields_ = [("vocab_size", C.c_uint32), ("dim", C.c_uint32), ("num_heads", C.c_uint32),
                ("num_layers", C.c_uint32), ("seq_len", C.c_uint32), ("ffn_hidden", C.c_uint32),
                ("norm_eps", C.c_float), ("eos_token", C.c_uint32)]


def _u32struct(name, fields, floats=()):
    return type(name, (C.Structure,), {"_fields_": [(f, C.c_float if f in floats else C.c_uint32) for f in fields]})


MatMulMeta = _u32struct("MatMulMeta", ["m", "n", "k"])
NormMeta = _u32struct("NormMeta", ["seq_len", "size", "eps"], floats=("eps",))
HeadMoveMeta = _u32struct("HeadMoveMeta", ["seq_len", "full_dim", "head_dim", "head_offset"])
AttnCachedMeta = _u32struct("AttnCachedMeta", ["attn_len", "dim", "head_dim"])
SoftmaxRectMeta = _u32struct("SoftmaxRectMeta", ["num_rows", "width", "scale"], floats=("scale",))
RopeMeta = _u32struct("RopeMeta", ["seq_len", "dim", "head_dim", "row_offset"])
RopeOffsetMeta = _u32struct("RopeOffsetMeta", ["seq_len", "dim", "head_dim", "pos"])
CacheWriteMeta = _u32struct("CacheWriteMeta", ["row_count", "width", "dst_row_offset"])
EmbeddingMeta = _u32struct("EmbeddingMeta", ["vocab_size", "dim", "seq_len"])
FlashAttnMeta = _u32struct("FlashAttnMeta", ["seq_len", "dim", "head_dim", "scale", "row_offset"], floats=("scale",))
AttnDecodeParams = _u32struct("AttnDecodeParams", ["rows", "heads", "head_dim", "block_size", "max_blocks_per_seq",
                                                   "scale", "kv_dtype", "n_splits", "pool_blocks"], floats=("scale",))
EngineConfig = _u32struct("EngineConfig", ["max_seqs", "max_seq_len", "kv_blocks", "block_size", "max_batch_tokens",
                                           "use_cuda_graph", "stop_on_eos", "attn_timing", "async_steps", "prefill_chunk_rows"])


class EngineStats(C.Structure):
    _fields_ = [("steps", C.c_uint64), ("decode_tokens", C.c_uint64), ("prefill_tokens", C.c_uint64),
                ("graph_launches", C.c_uint64), ("eager_steps", C.c_uint64), ("kernel_launches", C.c_uint64),
                ("attn_ms_total", C.c_double), ("attn_launches_timed", C.c_uint64), ("attn_bytes_total", C.c_uint64),
                ("h2d_bytes", C.c_uint64), ("d2h_bytes", C.c_uint64),
                ("step_gpu_ms_total", C.c_double), ("launch_host_ms_total", C.c_double),
                ("decode_step_gpu_ms_total", C.c_double), ("decode_steps_timed", C.c_uint64),
                ("decode_step_bytes_total", C.c_uint64)]


# ------------------------------------------------------------------ library
_lib = None
vp, u32p, i32p, f32p = C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_int32), C.POINTER(C.c_float)

_PROTOS = {
    "ak_device_count": [C.POINTER(C.c_int)],
    "ak_set_device": [C.c_int],
    "ak_device_malloc": [C.POINTER(vp), C.c_size_t],
    "ak_device_free": [vp],
    "ak_memcpy_h2d": [vp, vp, C.c_size_t, vp],
    "ak_memcpy_d2h": [vp, vp, C.c_size_t, vp],
    "ak_memset": [vp, C.c_int, C.c_size_t, vp],
    "ak_stream_create": [C.POINTER(vp)],
    "ak_stream_destroy": [vp],
    "ak_stream_synchronize": [vp],
    "ak_host_alloc_pinned": [C.POINTER(vp), C.c_size_t],
    "ak_host_free_pinned": [vp],
    "ak_check_device_status": [vp],
    "ak_embedding": [vp, vp, vp, vp, EmbeddingMeta],
    "ak_rmsnorm": [vp, vp, vp, vp, NormMeta],
    "ak_matmul": [vp, vp, vp, vp, MatMulMeta],
    "ak_matmul_add": [vp, vp, vp, vp, MatMulMeta],
    "ak_head_gather": [vp, vp, vp, HeadMoveMeta],
    "ak_rope": [vp, vp, RopeMeta],
    "ak_rope_offset": [vp, vp, RopeOffsetMeta],
    "ak_cache_write": [vp, vp, vp, CacheWriteMeta],
    "ak_attn_qk_cached": [vp, vp, vp, vp, AttnCachedMeta],
    "ak_softmax_rect": [vp, vp, SoftmaxRectMeta],
    "ak_attn_av_cached": [vp, vp, vp, vp, AttnCachedMeta],
    "ak_flash_attention": [vp, vp, vp, vp, vp, vp, FlashAttnMeta],
    "ak_silu": [vp, vp, C.c_uint32],
    "ak_argmax": [vp, vp, C.c_uint32, C.c_uint32, vp],
    "ak_sample_token": [vp, vp, C.c_uint32, C.c_uint32, vp, vp, C.c_float, C.c_float, C.c_uint32, C.c_float, C.c_uint64, C.c_uint64, vp],
    "ak_attn_decode_paged": [vp, vp, vp, vp, vp, vp, vp, vp, AttnDecodeParams],
    "ak_attn_decode_paged_noalloc": [vp, vp, vp, vp, vp, vp, vp, AttnDecodeParams],
    "ak_attn_decode_append_paged": [vp, vp, vp, C.c_uint32, vp, vp, vp, vp, vp, vp, AttnDecodeParams],
    "ak_attn_prefill_paged": [vp, vp, vp, vp, vp, C.c_uint32, vp, vp, vp] + [C.c_uint32] * 5 + [C.c_float, C.c_uint32, C.c_uint32],
    "ak_rope_kv_append": [vp, vp, vp, vp, vp, vp, vp] + [C.c_uint32] * 5,
    "ak_rmsnorm_rope_residual": [vp, vp, vp, vp, vp, vp, C.c_uint32, C.c_uint32, C.c_float, C.c_uint32, C.c_uint32],
    "ak_gemm_bf16": [vp, vp, vp, vp, MatMulMeta, C.c_uint32],
    "ak_gemm_bf16_ld": [vp, vp, vp, vp, MatMulMeta, C.c_uint32, C.c_uint32],
    "ak_transpose_to_bf16": [vp, vp, vp, C.c_uint32, C.c_uint32],
    "ak_f32_to_bf16": [vp, vp, vp, C.c_uint64],
    "ak_bf16_to_f32": [vp, vp, vp, C.c_uint64],
    "ak_ctx_create": [C.c_int, C.POINTER(vp)],
    "ak_ctx_destroy": [vp],
    "ak_ctx_synchronize": [vp],
    "ak_tp_unique_id": [vp],
    "ak_ctx_tp_init": [vp, C.c_uint32, C.c_uint32, vp],
    "ak_ctx_tp_shutdown": [vp],
    "ak_weights_create": [vp, C.POINTER(_ModelConfig), C.c_uint32, C.POINTER(vp)],
    "ak_weights_destroy": [vp],
    "ak_weights_set_param": [vp, C.c_uint32, f32p, C.c_uint64],
    "ak_weights_get_param": [vp, C.c_uint32, f32p, C.c_uint64],
    "ak_weights_init_synthetic": [vp, C.c_uint64, C.c_float],
    "ak_akv3_read_header": [C.c_char_p, C.POINTER(_ModelConfig), C.POINTER(C.c_uint64)],
    "ak_weights_load_akv3": [vp, C.c_char_p, C.POINTER(C.c_uint64)],
    "ak_session_create": [vp, vp, C.c_uint32, C.POINTER(vp)],
    "ak_session_destroy": [vp],
    "ak_session_attach_cache": [vp],
    "ak_session_take_cache": [vp],
    "ak_session_reset_cache": [vp],
    "ak_session_prefill": [vp, u32p, C.c_uint32, f32p, u32p],
    "ak_session_decode_step": [vp, C.c_uint32, f32p, u32p],
    "ak_session_generate_greedy": [vp, u32p, C.c_uint32, C.c_uint32, C.c_int, u32p, u32p],
    "ak_session_read_cache": [vp, C.c_uint32, f32p, f32p],
    "ak_engine_create": [vp, vp, C.POINTER(EngineConfig), C.POINTER(vp)],
    "ak_engine_destroy": [vp],
    "ak_engine_submit": [vp, u32p, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64)],
    "ak_engine_step": [vp, u32p, u32p],
    "ak_engine_run": [vp, C.c_uint64, C.POINTER(C.c_uint64)],
    "ak_engine_poll": [vp, C.c_uint64, u32p, C.c_uint32, u32p, C.POINTER(C.c_int)],
    "ak_engine_block_table": [vp, C.c_uint64, i32p, C.c_uint32, u32p],
    "ak_engine_clear_finished": [vp],
    "ak_session_generate": [vp, u32p, C.c_uint32, C.c_uint32, C.c_float, C.c_uint32, C.c_float, C.c_float, C.c_uint64, C.c_int, u32p,
                            u32p],
    "ak_engine_get_stats": [vp, C.POINTER(EngineStats)],
    "ak_engine_reset_stats": [vp],
}


def lib() -> C.CDLL:
    """Load the CUDA library. Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python akasha-core_b200/build.py` "
                              "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        for name, args in _PROTOS.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = C.c_int
        L.ak_last_error_string.restype = C.c_char_p
        L.ak_version.restype = C.c_char_p
        L.ak_launch_count.restype = C.c_ulonglong
        L.ak_ctx_stream.argtypes = [vp]
        L.ak_ctx_stream.restype = vp
        L.ak_weights_param_count.argtypes = [vp]
        L.ak_weights_param_count.restype = C.c_uint32
        L.ak_weights_param_len.argtypes = [vp, C.c_uint32]
        L.ak_weights_param_len.restype = C.c_uint64
        L.ak_session_cur_len.argtypes = [vp]
        L.ak_session_cur_len.restype = C.c_uint32
        L.ak_attn_decode_scratch_bytes.argtypes = [C.POINTER(AttnDecodeParams)]
        L.ak_attn_decode_scratch_bytes.restype = C.c_size_t
        L.ak_attn_decode_noalloc_max_scratch_bytes.argtypes = []
        L.ak_attn_decode_noalloc_max_scratch_bytes.restype = C.c_size_t
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise AkashaError(rc, lib().ak_last_error_string().decode())


def launch_count() -> int:
    return int(lib().ak_launch_count())


# ------------------------------------------------------------------ config
@dataclass(frozen=True)
class ModelConfig:
    """`ModelConfig::new` (src/config.rs:15-30): ffn = 4*dim, eps = 1e-5, eos = vocab-1."""
    vocab_size: int
    dim: int
    num_heads: int
    num_layers: int
    seq_len: int
    ffn_hidden: int = 0
    norm_eps: float = 1e-5
    eos_token: int = -1

    def __post_init__(self):
        assert self.num_layers >= 1, "At least one layer is required!"
        assert self.dim % self.num_heads == 0, "dim must be divisible by num_heads"
        if self.ffn_hidden == 0:
            object.__setattr__(self, "ffn_hidden", 4 * self.dim)
        if self.eos_token < 0:
            object.__setattr__(self, "eos_token", self.vocab_size - 1)

    @property
    def head_dim(self) -> int:
        return self.dim // self.num_heads

    @staticmethod
    def akasha_hall_1() -> "ModelConfig":  # src/config.rs:54-56
        return ModelConfig(50257, 768, 12, 12, 512)

    @staticmethod
    def pidgeon() -> "ModelConfig":  # src/config.rs:58-60
        return ModelConfig(50257, 320, 5, 8, 512)

    @staticmethod
    def scaled_1p4b() -> "ModelConfig":
        """The scaled synthetic model: dim 2048, 24 layers, 16 heads x 128, ctx 4096."""
        return ModelConfig(50257, 2048, 16, 24, 4096)

    def param_shapes(self):
        """Shapes in `ModelWeights::params()` order (src/nn/weights.rs:158-171); matrices [in,out]."""
        V, D, F = self.vocab_size, self.dim, self.ffn_hidden
        shapes = [(V, D)]
        for _ in range(self.num_layers):
            shapes += [(D,), (D, 3 * D), (D, D), (D,), (D, F), (F, D)]
        shapes += [(D,), (D, V)]
        return shapes

    def as_dict(self):
        return dict(vocab_size=self.vocab_size, dim=self.dim, num_heads=self.num_heads, num_layers=self.num_layers,
                    seq_len=self.seq_len, ffn_hidden=self.ffn_hidden, norm_eps=self.norm_eps, eos_token=self.eos_token)

    def _c(self) -> _ModelConfig:
        return _ModelConfig(self.vocab_size, self.dim, self.num_heads, self.num_layers, self.seq_len,
                            self.ffn_hidden, self.norm_eps, self.eos_token)

    @property
    def n_params(self) -> int:
        return sum(int(np.prod(s)) for s in self.param_shapes())


def akv3_read_header(path: str):
    """(ModelConfig, train_step) of an AKV3 checkpoint file."""
    c, ts = _ModelConfig(), C.c_uint64(0)
    check(lib().ak_akv3_read_header(path.encode(), C.byref(c), C.byref(ts)))
    return ModelConfig(c.vocab_size, c.dim, c.num_heads, c.num_layers, c.seq_len, c.ffn_hidden, c.norm_eps, c.eos_token), ts.value


def akv3_write(path: str, cfg: "ModelConfig", params, train_step: int = 0, schedule_step: int = 0, moments=()):
    """Write an AKV3 file exactly as `checkpoint::save` lays it out (src/nn/checkpoint.rs:49-95).
    For tests and for exporting synthetic weights to the reference."""
    import struct
    with open(path, "wb") as f:
        f.write(b"AKV3")
        f.write(struct.pack("<IIIQIIQI", cfg.vocab_size, cfg.dim, cfg.num_heads, cfg.num_layers, cfg.seq_len,
                            cfg.ffn_hidden, train_step, schedule_step))
        f.write(struct.pack("<Q", len(params)))
        for p in params:
            a = np.ascontiguousarray(p, np.float32)
            f.write(struct.pack("<Q", a.size))
            f.write(a.tobytes())
        f.write(struct.pack("<Q", len(moments)))
        for m, v in moments:
            for t in (m, v):
                a = np.ascontiguousarray(t, np.float32)
                f.write(struct.pack("<Q", a.size))
                f.write(a.tobytes())


# ------------------------------------------------------------------ synthetic inputs
def _splitmix64(z: np.ndarray) -> np.ndarray:
    z = (z + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def normal_f32(n: int, seed: int, stream: int, mean: float, std: float) -> np.ndarray:
    """Counter-based N(mean, std): splitmix64(seed, stream, i) -> two 24-bit uniforms -> Box-Muller
    in float64, rounded once to float32."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.uint64(seed) ^ _splitmix64(np.array([stream * 0x632BE59BD9B4E019 + 1 & (2**64 - 1)], np.uint64)))[0]
        out = np.empty(n, np.float32)
        step = 1 << 22
        for s in range(0, n, step):
            e = min(n, s + step)
            r = _splitmix64(base + np.arange(s, e, dtype=np.uint64))
            u1 = (((r >> np.uint64(40)) & np.uint64(0xFFFFFF)).astype(np.float64) + 1.0) / 16777217.0
            u2 = ((r >> np.uint64(8)) & np.uint64(0xFFFFFF)).astype(np.float64) / 16777216.0
            out[s:e] = (mean + std * np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)
    return out


def synthetic_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02):
    """Seeded random-init weights in `params()` order: matrices ~ N(0, std), norm gains ~ N(1, std)
    (the reference's init draws gains around 1, src/nn/weights.rs:85,94,109)."""
    out = []
    for i, shp in enumerate(cfg.param_shapes()):
        n = int(np.prod(shp))
        mean = 1.0 if len(shp) == 1 else 0.0
        out.append(normal_f32(n, seed, i, mean, std).reshape(shp))
    return out


def uniform_tokens(n: int, vocab: int, seed: int) -> np.ndarray:
    """n token ids uniform in [0, vocab) from `seed`."""
    with np.errstate(over="ignore"):
        r = _splitmix64(np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15) + np.arange(n, dtype=np.uint64))
    return (r % np.uint64(vocab)).astype(np.uint32)


def uniform_ints(n: int, lo: int, hi: int, seed: int) -> np.ndarray:
    """n integers uniform in [lo, hi] (inclusive) from `seed`."""
    with np.errstate(over="ignore"):
        r = _splitmix64(np.uint64(seed) * np.uint64(0xD1B54A32D192ED03) + np.arange(n, dtype=np.uint64))
    return (np.uint64(lo) + r % np.uint64(hi - lo + 1)).astype(np.int64)


# ------------------------------------------------------------------ handles
class Context:
    """One device + one stream (the reference's `Arc<B: Backend>`; `CudaBackend::new(0)`)."""

    def __init__(self, device: int = 0):
        self.h = vp()
        check(lib().ak_ctx_create(device, C.byref(self.h)))
        self.device = device

    @property
    def stream(self):
        return lib().ak_ctx_stream(self.h)

    def synchronize(self):
        check(lib().ak_ctx_synchronize(self.h))

    @staticmethod
    def tp_unique_id() -> bytes:
        """128-byte NCCL id made by tensor-parallel rank 0; hand it to the other ranks."""
        buf = C.create_string_buffer(128)
        check(lib().ak_tp_unique_id(buf))
        return buf.raw

    def tp_init(self, tp_size: int, tp_rank: int, unique_id: bytes):
        """Join a tensor-parallel group; call before creating weights on this context."""
        assert len(unique_id) == 128
        check(lib().ak_ctx_tp_init(self.h, tp_size, tp_rank, C.create_string_buffer(unique_id, 128)))
        self.tp_size, self.tp_rank = tp_size, tp_rank

    def check_device_status(self):
        check(lib().ak_check_device_status(self.stream))

    def close(self):
        if self.h:
            lib().ak_ctx_destroy(self.h)
            self.h = None


class ModelWeights:
    """Device weights in the shared `ModelWeights` layout (src/nn/weights.rs:32-47)."""

    def __init__(self, ctx: Context, cfg: ModelConfig, dtype: int = AK_F32):
        self.ctx, self.cfg, self.dtype = ctx, cfg, dtype
        self.h = vp()
        c = cfg._c()
        check(lib().ak_weights_create(ctx.h, C.byref(c), dtype, C.byref(self.h)))

    @classmethod
    def from_params(cls, ctx, cfg, params, dtype=AK_F32):
        w = cls(ctx, cfg, dtype)
        w.load(params)
        return w

    def load(self, params):
        """`copy_from_cpu` per tensor in `params()` order (src/nn/checkpoint.rs:98-161)."""
        assert len(params) == lib().ak_weights_param_count(self.h)
        for i, p in enumerate(params):
            a = np.ascontiguousarray(p, np.float32)
            check(lib().ak_weights_set_param(self.h, i, a.ctypes.data_as(f32p), a.size))

    def load_akv3(self, path: str) -> int:
        """`checkpoint::load` (src/nn/checkpoint.rs:98-161): weights from an AKV3 file; returns train_step."""
        ts = C.c_uint64(0)
        check(lib().ak_weights_load_akv3(self.h, path.encode(), C.byref(ts)))
        return ts.value

    def init_synthetic(self, seed=0, std=0.02):
        check(lib().ak_weights_init_synthetic(self.h, seed, std))

    def params(self):
        out = []
        for i, shp in enumerate(self.cfg.param_shapes()):
            a = np.empty(shp, np.float32)
            check(lib().ak_weights_get_param(self.h, i, a.ctypes.data_as(f32p), a.size))
            out.append(a)
        return out

    def close(self):
        if self.h:
            lib().ak_weights_destroy(self.h)
            self.h = None


class InferenceSession:
    """Mirror of `InferenceSession` (src/nn/inference.rs:13-327). Logits come back as numpy f32."""

    def __init__(self, ctx: Context, weights: ModelWeights, max_context_len: int):
        self.ctx, self.weights, self.max_context_len = ctx, weights, max_context_len
        self.h = vp()
        check(lib().ak_session_create(ctx.h, weights.h, max_context_len, C.byref(self.h)))
        self._V = weights.cfg.vocab_size

    def replace_cache(self):
        """`replace_cache(Cache::new(..))`: attach a fresh, empty cache."""
        check(lib().ak_session_attach_cache(self.h))

    def take_cache(self):
        check(lib().ak_session_take_cache(self.h))

    def reset_cache(self):
        check(lib().ak_session_reset_cache(self.h))

    @property
    def cur_len(self) -> int:
        return lib().ak_session_cur_len(self.h)

    def prefill(self, prompt_tokens, want_logits=True):
        t = np.ascontiguousarray(prompt_tokens, np.uint32)
        logits = np.empty(self._V, np.float32) if want_logits else None
        am = C.c_uint32(0)
        check(lib().ak_session_prefill(self.h, t.ctypes.data_as(u32p), t.size,
                                       logits.ctypes.data_as(f32p) if want_logits else None, C.byref(am)))
        return (logits, am.value) if want_logits else am.value

    def decode_step(self, token: int, want_logits=True):
        logits = np.empty(self._V, np.float32) if want_logits else None
        am = C.c_uint32(0)
        check(lib().ak_session_decode_step(self.h, int(token), logits.ctypes.data_as(f32p) if want_logits else None,
                                           C.byref(am)))
        return (logits, am.value) if want_logits else am.value

    def generate(self, prompt_tokens, max_new_tokens: int, stop_on_eos: bool = True, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, repetition_penalty: float = 1.0, seed: int = 0):
        """`generate` (src/nn/inference.rs:264-326); returns token ids. With the defaults it is the greedy
        path (temperature <= 0, repetition_penalty == 1); any other setting samples on the device with
        `sample_token`'s rules (`run_chat` uses 0.8, 40, 0.95, 1.15)."""
        t = np.ascontiguousarray(prompt_tokens, np.uint32)
        out = np.zeros(max(1, max_new_tokens), np.uint32)
        n = C.c_uint32(0)
        if temperature <= 0.0 and repetition_penalty == 1.0:
            check(lib().ak_session_generate_greedy(self.h, t.ctypes.data_as(u32p), t.size, max_new_tokens,
                                                   int(stop_on_eos), out.ctypes.data_as(u32p), C.byref(n)))
        else:
            check(lib().ak_session_generate(self.h, t.ctypes.data_as(u32p), t.size, max_new_tokens, temperature, top_k, top_p,
                                            repetition_penalty, seed, int(stop_on_eos), out.ctypes.data_as(u32p), C.byref(n)))
        return out[:n.value].copy()

    def read_cache(self, layer: int):
        n, D = self.cur_len, self.weights.cfg.dim
        k = np.empty((n, D), np.float32)
        v = np.empty((n, D), np.float32)
        check(lib().ak_session_read_cache(self.h, layer, k.ctypes.data_as(f32p), v.ctypes.data_as(f32p)))
        return k, v

    def close(self):
        if self.h:
            lib().ak_session_destroy(self.h)
            self.h = None


class Engine:
    """Continuous batching over the paged KV cache."""

    def __init__(self, ctx: Context, weights: ModelWeights, max_seqs: int, max_seq_len: int, kv_blocks: int = 0,
                 max_batch_tokens: int = 0, use_cuda_graph: bool = True, stop_on_eos: bool = False,
                 attn_timing: bool = False, async_steps: bool = False, prefill_chunk_rows: int = 0):
        self.ctx, self.weights = ctx, weights
        cfg = EngineConfig(max_seqs, max_seq_len, kv_blocks, 16, max_batch_tokens, int(use_cuda_graph),
                           int(stop_on_eos), int(attn_timing), int(async_steps), int(prefill_chunk_rows))
        self.h = vp()
        check(lib().ak_engine_create(ctx.h, weights.h, C.byref(cfg), C.byref(self.h)))

    def submit(self, prompt, max_total_len: int) -> int:
        t = np.ascontiguousarray(prompt, np.uint32)
        sid = C.c_uint64(0)
        check(lib().ak_engine_submit(self.h, t.ctypes.data_as(u32p), t.size, max_total_len, C.byref(sid)))
        return sid.value

    def step(self):
        r, w = C.c_uint32(0), C.c_uint32(0)
        check(lib().ak_engine_step(self.h, C.byref(r), C.byref(w)))
        return r.value, w.value

    def run_to_completion(self, max_steps: int = 1 << 30) -> int:
        """Step until nothing is running or waiting (the loop runs inside the library)."""
        n = C.c_uint64(0)
        check(lib().ak_engine_run(self.h, max_steps, C.byref(n)))
        return n.value

    def poll(self, seq_id: int, cap: int = 8192):
        out = np.zeros(cap, np.uint32)
        n, fin = C.c_uint32(0), C.c_int(0)
        check(lib().ak_engine_poll(self.h, seq_id, out.ctypes.data_as(u32p), cap, C.byref(n), C.byref(fin)))
        return out[:min(n.value, cap)].copy(), bool(fin.value)

    def block_table(self, seq_id: int, cap: int = 4096):
        out = np.zeros(cap, np.int32)
        n = C.c_uint32(0)
        check(lib().ak_engine_block_table(self.h, seq_id, out.ctypes.data_as(i32p), cap, C.byref(n)))
        return out[:n.value].copy()

    def clear_finished(self):
        check(lib().ak_engine_clear_finished(self.h))

    def stats(self) -> dict:
        s = EngineStats()
        check(lib().ak_engine_get_stats(self.h, C.byref(s)))
        return {f: getattr(s, f) for f, _ in EngineStats._fields_}

    def reset_stats(self):
        check(lib().ak_engine_reset_stats(self.h))

    def close(self):
        if self.h:
            lib().ak_engine_destroy(self.h)
            self.h = None


from . import ops  # noqa: E402  (emitter-level functions)
