//! `extern "C"` declarations for every symbol `include/akasha_b200.h` exports.
#![allow(non_camel_case_types)]
use crate::meta::*;
use std::os::raw::{c_char, c_int, c_ulonglong, c_void};

pub const AK_F32: u32 = 0;
pub const AK_BF16: u32 = 1;

// return codes (ak_status): 1..5 = AkashaError in declaration order (src/lib.rs:10-17)
pub const AK_OK: c_int = 0;
pub const AK_EMPTY_PROMPT: c_int = 1;
pub const AK_PROMPT_TOO_LONG: c_int = 2;
pub const AK_CONTEXT_FULL: c_int = 3;
pub const AK_NO_CACHE: c_int = 4;
pub const AK_CACHE_NOT_EMPTY: c_int = 5;
pub const AK_ERR_INVALID_ARG: c_int = 100;
pub const AK_ERR_CUDA: c_int = 101;
pub const AK_ERR_ALLOC: c_int = 102;
pub const AK_ERR_UNSUPPORTED: c_int = 103;
pub const AK_ERR_DEVICE_WAIT: c_int = 104;
pub const AK_ERR_NO_CAPACITY: c_int = 105;
pub const AK_ERR_NOT_FOUND: c_int = 106;

// ak_gemm_epilogue
pub const AK_EPI_STORE_F32: u32 = 0;
pub const AK_EPI_ADD_F32: u32 = 1;
pub const AK_EPI_STORE_BF16: u32 = 2;
pub const AK_EPI_SILU_BF16: u32 = 3;

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct AkModelConfig {
    pub vocab_size: u32,
    pub dim: u32,
    pub num_heads: u32,
    pub num_layers: u32,
    pub seq_len: u32,
    pub ffn_hidden: u32,
    pub norm_eps: f32,
    pub eos_token: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct AkAttnDecodeParams {
    pub rows: u32,
    pub heads: u32,
    pub head_dim: u32,
    pub block_size: u32,
    pub max_blocks_per_seq: u32,
    pub scale: f32,
    pub kv_dtype: u32,
    pub n_splits: u32,
    pub pool_blocks: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct AkEngineConfig {
    pub max_seqs: u32,
    pub max_seq_len: u32,
    pub kv_blocks: u32,
    pub block_size: u32,
    pub max_batch_tokens: u32,
    pub use_cuda_graph: u32,
    pub stop_on_eos: u32,
    pub attn_timing: u32,
    pub async_steps: u32,
    pub prefill_chunk_rows: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct AkEngineStats {
    pub steps: u64,
    pub decode_tokens: u64,
    pub prefill_tokens: u64,
    pub graph_launches: u64,
    pub eager_steps: u64,
    pub kernel_launches: u64,
    pub attn_ms_total: f64,
    pub attn_launches_timed: u64,
    pub attn_bytes_total: u64,
    pub h2d_bytes: u64,
    pub d2h_bytes: u64,
    pub step_gpu_ms_total: f64,
    pub launch_host_ms_total: f64,
    pub decode_step_gpu_ms_total: f64,
    pub decode_steps_timed: u64,
    pub decode_step_bytes_total: u64,
}

macro_rules! opaque { ($($n:ident),*) => { $(#[repr(C)] pub struct $n { _p: [u8; 0] })* }; }
opaque!(AkCtx, AkWeights, AkSession, AkEngine);

pub type Stream = *mut c_void;

extern "C" {
    // ---- library, device, streams, memory
    pub fn ak_last_error_string() -> *const c_char;
    pub fn ak_version() -> *const c_char;
    pub fn ak_launch_count() -> c_ulonglong;
    pub fn ak_check_device_status(stream: Stream) -> c_int;
    pub fn ak_device_count(out: *mut c_int) -> c_int;
    pub fn ak_set_device(device: c_int) -> c_int;
    pub fn ak_device_malloc(out: *mut *mut c_void, bytes: usize) -> c_int;
    pub fn ak_device_free(p: *mut c_void) -> c_int;
    pub fn ak_memcpy_h2d(dst: *mut c_void, src: *const c_void, bytes: usize, stream: Stream) -> c_int;
    pub fn ak_memcpy_d2h(dst: *mut c_void, src: *const c_void, bytes: usize, stream: Stream) -> c_int;
    pub fn ak_memset(dst: *mut c_void, value: c_int, bytes: usize, stream: Stream) -> c_int;
    pub fn ak_stream_create(out: *mut Stream) -> c_int;
    pub fn ak_stream_destroy(stream: Stream) -> c_int;
    pub fn ak_stream_synchronize(stream: Stream) -> c_int;
    pub fn ak_host_alloc_pinned(out: *mut *mut c_void, bytes: usize) -> c_int;
    pub fn ak_host_free_pinned(p: *mut c_void) -> c_int;

    // ---- emitter level: device pointers + the crate's meta by value (src/nn/ops/emit.rs)
    pub fn ak_embedding(stream: Stream, tokens: *const u32, table: *const f32, out: *mut f32, m: EmbeddingMeta) -> c_int;
    pub fn ak_rmsnorm(stream: Stream, x: *const f32, w: *const f32, y: *mut f32, m: NormMeta) -> c_int;
    pub fn ak_matmul(stream: Stream, a: *const f32, b: *const f32, c: *mut f32, m: MatMulMeta) -> c_int;
    pub fn ak_matmul_add(stream: Stream, a: *const f32, b: *const f32, c: *mut f32, m: MatMulMeta) -> c_int;
    pub fn ak_head_gather(stream: Stream, src: *const f32, dst: *mut f32, m: HeadMoveMeta) -> c_int;
    pub fn ak_rope(stream: Stream, x: *mut f32, m: RopeMeta) -> c_int;
    pub fn ak_rope_offset(stream: Stream, x: *mut f32, m: RopeOffsetMeta) -> c_int;
    pub fn ak_cache_write(stream: Stream, src: *const f32, cache: *mut f32, m: CacheWriteMeta) -> c_int;
    pub fn ak_attn_qk_cached(stream: Stream, q: *const f32, k_cache: *const f32, scores: *mut f32, m: AttnCachedMeta) -> c_int;
    pub fn ak_softmax_rect(stream: Stream, x: *mut f32, m: SoftmaxRectMeta) -> c_int;
    pub fn ak_attn_av_cached(stream: Stream, scores: *const f32, v_cache: *const f32, out: *mut f32, m: AttnCachedMeta) -> c_int;
    pub fn ak_flash_attention(stream: Stream, q: *const f32, k: *const f32, v: *const f32, out: *mut f32, l_cache: *mut f32,
                              m: FlashAttnMeta) -> c_int;
    pub fn ak_silu(stream: Stream, x: *mut f32, n: u32) -> c_int;
    pub fn ak_argmax(stream: Stream, logits: *const f32, rows: u32, n: u32, out_idx: *mut u32) -> c_int;
    pub fn ak_sample_token(stream: Stream, logits: *const f32, rows: u32, n: u32, seen: *const u32, seen_off: *const u32,
                           repetition_penalty: f32, temperature: f32, top_k: u32, top_p: f32, seed: u64, step: u64,
                           out_idx: *mut u32) -> c_int;

    // ---- fused sm_100a kernels
    pub fn ak_attn_decode_scratch_bytes(p: *const AkAttnDecodeParams) -> usize;
    pub fn ak_attn_decode_paged(stream: Stream, q: *const c_void, k_pool: *const c_void, v_pool: *const c_void,
                                block_tables: *const i32, kv_lens: *const i32, out: *mut c_void, scratch: *mut c_void,
                                p: AkAttnDecodeParams) -> c_int;
    pub fn ak_attn_decode_append_paged(stream: Stream, qkv: *const f32, rope_table: *const f32, rope_len: u32, k_pool: *mut c_void,
                                       v_pool: *mut c_void, block_tables: *const i32, kv_lens: *const i32, out: *mut c_void,
                                       scratch: *mut c_void, p: AkAttnDecodeParams) -> c_int;
    pub fn ak_attn_decode_noalloc_max_scratch_bytes() -> usize;
    pub fn ak_attn_decode_paged_noalloc(stream: Stream, q: *const c_void, k_pool: *const c_void, v_pool: *const c_void,
                                        block_tables: *const i32, kv_lens: *const i32, out: *mut c_void,
                                        p: AkAttnDecodeParams) -> c_int;
    pub fn ak_rope_kv_append(stream: Stream, qkv: *const f32, positions: *const i32, slots: *const i32, q_out: *mut c_void,
                             k_pool: *mut c_void, v_pool: *mut c_void, tokens: u32, heads: u32, head_dim: u32, block_size: u32,
                             kv_dtype: u32) -> c_int;
    pub fn ak_attn_prefill_paged(stream: Stream, q: *const c_void, k_pool: *const c_void, v_pool: *const c_void,
                                 block_tables: *const i32, max_blocks_per_seq: u32, cu: *const i32, seq_slot: *const i32,
                                 out: *mut c_void, n_seqs: u32, max_len: u32, q_rows: u32, heads: u32, head_dim: u32, scale: f32,
                                 dtype: u32, pool_blocks: u32) -> c_int;
    pub fn ak_rmsnorm_rope_residual(stream: Stream, x: *mut f32, residual: *const f32, w: *const f32, y: *mut c_void,
                                    positions: *const i32, rows: u32, size: u32, eps: f32, head_dim: u32, out_dtype: u32) -> c_int;
    pub fn ak_gemm_bf16(stream: Stream, a: *const c_void, wt: *const c_void, c: *mut c_void, m: MatMulMeta, epilogue: u32) -> c_int;
    pub fn ak_gemm_bf16_ld(stream: Stream, a: *const c_void, wt: *const c_void, c: *mut c_void, m: MatMulMeta, epilogue: u32,
                           ldc: u32) -> c_int;
    pub fn ak_transpose_to_bf16(stream: Stream, w_kn: *const f32, wt_nk: *mut c_void, k: u32, n: u32) -> c_int;
    pub fn ak_f32_to_bf16(stream: Stream, src: *const f32, dst: *mut c_void, n: u64) -> c_int;
    pub fn ak_bf16_to_f32(stream: Stream, src: *const c_void, dst: *mut f32, n: u64) -> c_int;

    // ---- context, tensor parallelism, weights (`ModelWeights::params()` order, src/nn/weights.rs:158-171)
    pub fn ak_ctx_create(device: c_int, out: *mut *mut AkCtx) -> c_int;
    pub fn ak_ctx_destroy(ctx: *mut AkCtx) -> c_int;
    pub fn ak_ctx_synchronize(ctx: *mut AkCtx) -> c_int;
    pub fn ak_ctx_stream(ctx: *mut AkCtx) -> Stream;
    pub fn ak_tp_unique_id(out128: *mut c_void) -> c_int;
    pub fn ak_ctx_tp_init(ctx: *mut AkCtx, tp_size: u32, tp_rank: u32, unique_id128: *const c_void) -> c_int;
    pub fn ak_ctx_tp_shutdown(ctx: *mut AkCtx) -> c_int;
    pub fn ak_weights_create(ctx: *mut AkCtx, cfg: *const AkModelConfig, dtype: u32, out: *mut *mut AkWeights) -> c_int;
    pub fn ak_weights_destroy(w: *mut AkWeights) -> c_int;
    pub fn ak_weights_param_count(w: *const AkWeights) -> u32;
    pub fn ak_weights_param_len(w: *const AkWeights, index: u32) -> u64;
    pub fn ak_weights_set_param(w: *mut AkWeights, index: u32, host: *const f32, n_elems: u64) -> c_int;
    pub fn ak_weights_get_param(w: *mut AkWeights, index: u32, host: *mut f32, n_elems: u64) -> c_int;
    pub fn ak_weights_init_synthetic(w: *mut AkWeights, seed: u64, std: f32) -> c_int;
    pub fn ak_akv3_read_header(path: *const c_char, cfg_out: *mut AkModelConfig, train_step_out: *mut u64) -> c_int;
    pub fn ak_weights_load_akv3(w: *mut AkWeights, path: *const c_char, train_step_out: *mut u64) -> c_int;

    // ---- session level (`InferenceSession`, src/nn/inference.rs:13-327)
    pub fn ak_session_create(ctx: *mut AkCtx, w: *mut AkWeights, max_context_len: u32, out: *mut *mut AkSession) -> c_int;
    pub fn ak_session_destroy(s: *mut AkSession) -> c_int;
    pub fn ak_session_attach_cache(s: *mut AkSession) -> c_int;
    pub fn ak_session_take_cache(s: *mut AkSession) -> c_int;
    pub fn ak_session_reset_cache(s: *mut AkSession) -> c_int;
    pub fn ak_session_cur_len(s: *const AkSession) -> u32;
    pub fn ak_session_prefill(s: *mut AkSession, tokens: *const u32, n: u32, logits_out: *mut f32, argmax_out: *mut u32) -> c_int;
    pub fn ak_session_decode_step(s: *mut AkSession, token: u32, logits_out: *mut f32, argmax_out: *mut u32) -> c_int;
    pub fn ak_session_generate_greedy(s: *mut AkSession, prompt: *const u32, n: u32, max_new: u32, stop_on_eos: c_int,
                                      out_tokens: *mut u32, n_out: *mut u32) -> c_int;
    pub fn ak_session_generate(s: *mut AkSession, prompt: *const u32, n: u32, max_new: u32, temperature: f32, top_k: u32, top_p: f32,
                               repetition_penalty: f32, seed: u64, stop_on_eos: c_int, out_tokens: *mut u32, n_out: *mut u32) -> c_int;
    pub fn ak_session_read_cache(s: *mut AkSession, layer: u32, k_out: *mut f32, v_out: *mut f32) -> c_int;

    // ---- engine level (continuous batching)
    pub fn ak_engine_create(ctx: *mut AkCtx, w: *mut AkWeights, cfg: *const AkEngineConfig, out: *mut *mut AkEngine) -> c_int;
    pub fn ak_engine_destroy(e: *mut AkEngine) -> c_int;
    pub fn ak_engine_submit(e: *mut AkEngine, prompt: *const u32, n: u32, max_total_len: u32, seq_id: *mut u64) -> c_int;
    pub fn ak_engine_step(e: *mut AkEngine, n_running: *mut u32, n_waiting: *mut u32) -> c_int;
    pub fn ak_engine_run(e: *mut AkEngine, max_steps: u64, steps_done: *mut u64) -> c_int;
    pub fn ak_engine_poll(e: *mut AkEngine, seq_id: u64, out: *mut u32, cap: u32, n_out: *mut u32, finished: *mut c_int) -> c_int;
    pub fn ak_engine_block_table(e: *mut AkEngine, seq_id: u64, out: *mut i32, cap: u32, n_out: *mut u32) -> c_int;
    pub fn ak_engine_clear_finished(e: *mut AkEngine) -> c_int;
    pub fn ak_engine_get_stats(e: *mut AkEngine, out: *mut AkEngineStats) -> c_int;
    pub fn ak_engine_reset_stats(e: *mut AkEngine) -> c_int;
}
