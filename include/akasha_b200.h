/*
 * akasha_b200.h -- C ABI of the B200 (sm_100a) backend for the akasha-hall Prefill/Decode
 * inference path.
 *
 * Three levels, all `extern "C"`, plain pointers and sizes only:
 *   1. emitter level  -- one entry point per forward/cached kernel emitter of the reference's
 *                        `src/nn/ops/emit.rs`, taking DEVICE pointers and the same `#[repr(C)]`
 *                        meta struct (by value) that `src/nn/ops/meta.rs` defines; plus the new
 *                        fused B200 kernels (paged decode attention, tcgen05 GEMM, ...).
 *   2. session level  -- mirrors `InferenceSession` (src/nn/inference.rs:13-327).
 *   3. engine level   -- continuous batching over a paged KV cache (new: the reference has no
 *                        batching, ARCHITECTURE.md:376-377).
 *
 * Every function returns an `ak_status`; 0 is success. Codes 1..5 mirror `AkashaError`
 * (src/lib.rs:10-17) in declaration order. Nothing here aborts the process, and no device code
 * traps: device-side waits are bounded and report through a status word.
 *
 * `stream` arguments are a `cudaStream_t` passed as `void*` (NULL = the default stream).
 * No handle is thread-safe; calls on one handle must be serialised by the caller
 * (the reference API is `&mut self`, src/nn/inference.rs:61,178).
 */
#ifndef AKASHA_B200_H
#define AKASHA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define AK_API __attribute__((visibility("default")))
#else
#define AK_API
#endif

/* ------------------------------------------------------------------ status */
typedef enum ak_status {
    AK_OK = 0,
    AK_EMPTY_PROMPT = 1,    /* AkashaError::EmptyPrompt    (src/lib.rs:12) */
    AK_PROMPT_TOO_LONG = 2, /* AkashaError::PromptTooLong  (src/lib.rs:13) */
    AK_CONTEXT_FULL = 3,    /* AkashaError::ContextFull    (src/lib.rs:14) */
    AK_NO_CACHE = 4,        /* AkashaError::NoCache        (src/lib.rs:15) */
    AK_CACHE_NOT_EMPTY = 5, /* AkashaError::CacheNotEmpty  (src/lib.rs:16) */
    AK_ERR_INVALID_ARG = 100,
    AK_ERR_CUDA = 101,
    AK_ERR_ALLOC = 102,
    AK_ERR_UNSUPPORTED = 103, /* shape / dtype the sm_100a kernels do not cover */
    AK_ERR_DEVICE_WAIT = 104, /* a bounded device-side wait ran out (status word set) */
    AK_ERR_NO_CAPACITY = 105, /* engine: no free sequence slot or KV block */
    AK_ERR_NOT_FOUND = 106
} ak_status;

/* Text of the last error raised on the calling thread ("" if none). */
AK_API const char* ak_last_error_string(void);
/* Library version string, and the compute architecture the kernels were built for. */
AK_API const char* ak_version(void);
/* Kernel launches issued by this library on the calling thread since it loaded. */
AK_API unsigned long long ak_launch_count(void);
/* Environment switches read by the library (both are measurement aids, off by default):
 *   AK_PDL=0    launch every kernel without the programmatic-dependent-launch attribute (A/B timing of the overlap);
 *   AK_TRACE=1  record an event after every launch of a step and print per-kernel in-stream times to stderr
 *               (the events remove the overlap between kernels, so the figures are upper bounds). */
/* Synchronise `stream` and read the device status words: AK_ERR_DEVICE_WAIT if a bounded
 * device-side wait (mbarrier / TMA / tcgen05 pipeline) ever ran out, AK_OK otherwise. */
AK_API int ak_check_device_status(void* stream);

/* ------------------------------------------------------------------ dtypes */
typedef enum ak_dtype {
    AK_F32 = 0, /* fp32 weights, KV and activations: the parity mode (true fp32 FMA everywhere) */
    AK_BF16 = 1 /* bf16 weights / KV / activations, fp32 accumulate and fp32 residual stream */
} ak_dtype;

/* ------------------------------------------------------------------ model config
 * ModelConfig (src/config.rs:2-30). ffn_hidden = 4*dim, norm_eps = 1e-5 and
 * eos_token = vocab_size-1 are what `ModelConfig::new` fixes; they are explicit fields here. */
typedef struct ak_model_config {
    uint32_t vocab_size;
    uint32_t dim;
    uint32_t num_heads;
    uint32_t num_layers;
    uint32_t seq_len; /* the model's nominal context (informational) */
    uint32_t ffn_hidden;
    float norm_eps;
    uint32_t eos_token;
} ak_model_config;

/* ------------------------------------------------------------------ typed kernel metas
 * Field-for-field the `#[repr(C)]` structs of src/nn/ops/meta.rs (all members 4 bytes). */
typedef struct ak_matmul_meta { uint32_t m, n, k; } ak_matmul_meta;                     /* meta.rs:19-25  */
typedef struct ak_norm_meta { uint32_t seq_len, size; float eps; } ak_norm_meta;        /* meta.rs:29-35  */
typedef struct ak_head_move_meta { uint32_t seq_len, full_dim, head_dim, head_offset; } ak_head_move_meta; /* meta.rs:40-47 */
typedef struct ak_attn_cached_meta { uint32_t attn_len, dim, head_dim; } ak_attn_cached_meta; /* meta.rs:62-68 */
typedef struct ak_softmax_rect_meta { uint32_t num_rows, width; float scale; } ak_softmax_rect_meta; /* meta.rs:72-78 */
typedef struct ak_rope_meta { uint32_t seq_len, dim, head_dim, row_offset; } ak_rope_meta; /* meta.rs:82-89 */
typedef struct ak_rope_offset_meta { uint32_t seq_len, dim, head_dim, pos; } ak_rope_offset_meta; /* meta.rs:93-100 */
typedef struct ak_cache_write_meta { uint32_t row_count, width, dst_row_offset; } ak_cache_write_meta; /* meta.rs:104-110 */
typedef struct ak_embedding_meta { uint32_t vocab_size, dim, seq_len; } ak_embedding_meta; /* meta.rs:114-120 */
typedef struct ak_flash_attn_meta { uint32_t seq_len, dim, head_dim; float scale; uint32_t row_offset; } ak_flash_attn_meta; /* meta.rs:156-164 */

/* ------------------------------------------------------------------ device helpers
 * For hosts that have no CUDA runtime binding of their own (the reference's Tensor::
 * init_from_cpu / copy_from_cpu / to_cpu, used at src/nn/inference.rs:83,189,261). */
AK_API int ak_device_count(int* out);
AK_API int ak_set_device(int device);
AK_API int ak_device_malloc(void** out, size_t bytes);
AK_API int ak_device_free(void* p);
AK_API int ak_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream);
AK_API int ak_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream);
AK_API int ak_memset(void* dst, int value, size_t bytes, void* stream);
AK_API int ak_stream_create(void** out);
AK_API int ak_stream_destroy(void* stream);
AK_API int ak_stream_synchronize(void* stream); /* ctx.synchronize(), src/nn/ops/emit.rs:1052 */
AK_API int ak_host_alloc_pinned(void** out, size_t bytes);
AK_API int ak_host_free_pinned(void* p);

/* ================================================================== 1. emitter level
 * All pointers are device pointers; f32 row-major as in the reference. Output-mode buffers are
 * fully overwritten, Accumulate-mode buffers are `+=` (ARCHITECTURE.md:226-231). */

/* ops::embedding (src/nn/ops/emit.rs:228-257; kernel src/shaders/cuda.rs:5-31):
 * out[t,:] = table[tokens[t],:], a zero row for an id >= vocab_size. */
AK_API int ak_embedding(void* stream, const uint32_t* tokens, const float* table, float* out, ak_embedding_meta m);
/* ops::rmsnorm (emit.rs:151-180; cuda.rs:421-456): y = x * rsqrt(mean(x^2)+eps) * w per row. */
AK_API int ak_rmsnorm(void* stream, const float* x, const float* w, float* y, ak_norm_meta m);
/* ops::matmul (emit.rs:23-57): C[m,n] = A[m,k] @ B[k,n]; m == 1 routes to the GEMV kernel. */
AK_API int ak_matmul(void* stream, const float* a, const float* b, float* c, ak_matmul_meta m);
/* ops::matmul_add (emit.rs:92-126): C[m,n] += A[m,k] @ B[k,n] (fused residual). */
AK_API int ak_matmul_add(void* stream, const float* a, const float* b, float* c, ak_matmul_meta m);
/* ops::head_gather (emit.rs:406-424; cuda.rs:256-274): dst[r,c] = src[r*full_dim+head_offset+c]. */
AK_API int ak_head_gather(void* stream, const float* src, float* dst, ak_head_move_meta m);
/* ops::rope (emit.rs:306-313; cuda.rs:98-123): in-place, adjacent pairs, position = row index. */
AK_API int ak_rope(void* stream, float* x, ak_rope_meta m);
/* ops::rope_offset_with (emit.rs:325-342; cuda.rs:224-254): position = row index + pos. */
AK_API int ak_rope_offset(void* stream, float* x, ak_rope_offset_meta m);
/* ops::cache_write (emit.rs:649-675; cuda.rs:614-631): cache[(off+r)*width+c] = src[r*width+c]. */
AK_API int ak_cache_write(void* stream, const float* src, float* cache, ak_cache_write_meta m);
/* ops::attn_qk_cached_with (emit.rs:485-504; cuda.rs:349-369): scores[h*attn_len+j] = q_h . K[j]_h (unscaled). */
AK_API int ak_attn_qk_cached(void* stream, const float* q, const float* k_cache, float* scores, ak_attn_cached_meta m);
/* ops::softmax_rect_with (emit.rs:528-542; cuda.rs:391-419): rows of softmax(scale*x), in place. */
AK_API int ak_softmax_rect(void* stream, float* x, ak_softmax_rect_meta m);
/* ops::attn_av_cached_with (emit.rs:507-525; cuda.rs:371-389): out[d] = sum_j P[d/hd, j] * V[j, d]. */
AK_API int ak_attn_av_cached(void* stream, const float* scores, const float* v_cache, float* out, ak_attn_cached_meta m);
/* ops::flash_attention (emit.rs:556-597; cuda.rs:633-685): causal attention over rows
 * row_offset..row_offset+seq_len of q/k/v [*, dim]; l_cache (may be NULL) = max + log(sum). */
AK_API int ak_flash_attention(void* stream, const float* q, const float* k, const float* v, float* out, float* l_cache, ak_flash_attn_meta m);
/* ops::silu (emit.rs:686-696; cuda.rs:57-65): x = x / (1 + exp(-x)) in place, any n < 2^32. */
AK_API int ak_silu(void* stream, float* x, uint32_t n);
/* sampling::argmax (src/nn/sampling.rs:83-91) on the device: for each of `rows` rows of `n`
 * logits the FIRST index holding the maximum. out_idx: device uint32[rows]. */
AK_API int ak_argmax(void* stream, const float* logits, uint32_t rows, uint32_t n, uint32_t* out_idx);

/* sampling::sample_token (src/nn/sampling.rs:18-81) on the device, one row per sequence:
 * repetition penalty over the DISTINCT ids of seen[seen_off[r] .. seen_off[r+1]) (positive logits
 * divided, the others multiplied), then temperature / top-k / top-p with f64 probabilities.
 * temperature <= 0 is greedy. top_k when sampling: 1..1024, or 0 (or >= n) = no truncation, the reference's
 * default (the candidate list is the whole row; the top-p cut and the draw are located by bisection on the logit
 * value instead of a 50k-element sort). The uniform draw is
 * splitmix64(seed, step, row) (the reference uses an unseeded generator); equal logits are ordered
 * by index (the reference's unstable sort leaves that order open). */
AK_API int ak_sample_token(void* stream, const float* logits, uint32_t rows, uint32_t n, const uint32_t* seen,
                           const uint32_t* seen_off, float repetition_penalty, float temperature, uint32_t top_k, float top_p,
                           uint64_t seed, uint64_t step, uint32_t* out_idx);

/* ---- new fused sm_100a kernels (no single-emitter counterpart in the reference) ---- */

/* Ragged paged decode attention: fuses attn_qk_cached + softmax_rect + attn_av_cached
 * (src/nn/inference_graphs.rs:428-456) for `rows` independent sequences in one launch.
 *   q, out      [rows, heads*head_dim]      (kv_dtype: f32 or bf16, same type for q/out/pools)
 *   k_pool/v_pool  [n_blocks, heads, block_size(16), head_dim]
 *   block_tables   int32 [rows, max_blocks_per_seq]; kv_lens int32 [rows] (0 = row skipped,
 *                  its output is zero-filled)
 *   slot(pos) = block_tables[row][pos/16]*16 + pos%16
 *   scratch: device buffer of ak_attn_decode_scratch_bytes() bytes, needed only when the
 *            launch splits sequences over several CTAs (n_splits > 1); may be NULL otherwise.
 *            It holds the splits' partial results and one arrival counter per (row, head); the
 *            call clears the counters itself, so the buffer may hold anything. The CTA that
 *            arrives last merges the partials inside the same launch (no second kernel).
 *   n_splits: 0 = let the library choose; at most 32. */
typedef struct ak_attn_decode_params {
    uint32_t rows, heads, head_dim, block_size, max_blocks_per_seq;
    float scale;
    uint32_t kv_dtype; /* ak_dtype */
    uint32_t n_splits;
    uint32_t pool_blocks; /* blocks in each pool; 0 = unknown (no range protection) */
} ak_attn_decode_params;
AK_API size_t ak_attn_decode_scratch_bytes(const ak_attn_decode_params* p);
AK_API int ak_attn_decode_paged(void* stream, const void* q, const void* k_pool, const void* v_pool,
                                const int32_t* block_tables, const int32_t* kv_lens, void* out,
                                void* scratch, ak_attn_decode_params p);

/* Decode attention with the step's head split, RoPE and cache append fused in (head_dim 64 or 128): for every row,
 * the new token's q | k | v come from qkv [rows, 3*heads*head_dim] f32 (the qkv projection's output), its position
 * is kv_lens[row] - 1 (kv_lens counts the new token) and its slot block_tables[row][pos/16]*16 + pos%16. The kernel
 * rotates q and k (head_gather x3 -> rope_offset x2, src/nn/inference_graphs.rs:385-412; adjacent pairs,
 * src/shaders/cuda.rs:224-254), stores K (post-RoPE) and V (raw) at that slot (cache_write x2,
 * inference_graphs.rs:413-426) and attends over positions 0..pos (inference_graphs.rs:428-456).
 * rope_table: float2 (cos, sin) [rope_len][head_dim/2] of angle = (float)pos / powf(10000, 2i/head_dim);
 * every position must be < rope_len. Rows with kv_lens == 0 are skipped (zero output, nothing appended). */
AK_API int ak_attn_decode_append_paged(void* stream, const float* qkv, const float* rope_table, uint32_t rope_len,
                                       void* k_pool, void* v_pool, const int32_t* block_tables, const int32_t* kv_lens,
                                       void* out, void* scratch, ak_attn_decode_params p);

/* The same attention for callers that cannot allocate device memory when they call it (a plugin
 * living inside another framework's memory pool, a loop that bans allocator calls after start-up,
 * a process whose free HBM has all gone to the KV pool). It has no counterpart in the reference.
 * The split-KV partials go to a buffer built into the library image instead of caller scratch:
 *   - each GPU that loads the library holds that buffer (ak_attn_decode_noalloc_max_scratch_bytes(),
 *     8 MiB) until the process exits;
 *   - a launch whose partials and counters (rows*heads*(n_splits*(head_dim+2)+1)*4 bytes) do not fit
 *     is refused with AK_ERR_UNSUPPORTED and a message; nothing is launched;
 *   - the call makes no cudaMalloc/cudaFree and calls no allocating library routine;
 *   - the first call on a device looks up the buffer's device address (that device must be
 *     current); make that first call before starting any stream capture;
 *   - all calls on one GPU share the buffer: calls that may overlap on the GPU (different streams)
 *     race on it and must be ordered by the caller. The buffer keeps the last call's contents:
 *     every partial that is read was written earlier in the same call, and the arrival counters,
 *     which must start at zero, are cleared on the stream by the call itself (a memset). */
AK_API size_t ak_attn_decode_noalloc_max_scratch_bytes(void);
AK_API int ak_attn_decode_paged_noalloc(void* stream, const void* q, const void* k_pool, const void* v_pool,
                                        const int32_t* block_tables, const int32_t* kv_lens, void* out,
                                        ak_attn_decode_params p);

/* Fused head split + RoPE + paged KV append (head_gather x3, rope(_offset) x2, cache_write x2:
 * src/nn/inference_graphs.rs:241-269, 385-426) over a ragged token batch.
 *   qkv [tokens, 3*dim] f32;  positions int32[tokens];  slots int32[tokens] (paged slot of the
 *   token, -1 = do not append);  q_out [tokens, dim];  pools as above (dtype = kv_dtype).
 * K is stored after RoPE, V raw (ARCHITECTURE.md:256-280). 128-bit stores throughout. */
AK_API int ak_rope_kv_append(void* stream, const float* qkv, const int32_t* positions, const int32_t* slots,
                             void* q_out, void* k_pool, void* v_pool, uint32_t tokens, uint32_t heads,
                             uint32_t head_dim, uint32_t block_size, uint32_t kv_dtype);

/* Causal attention of newly prefilled sequences over the paged KV pools: the prefill graph's
 * FLASH_ATTENTION node (src/nn/inference_graphs.rs:271-285, kernel src/shaders/cuda.rs:633-685)
 * for a ragged batch. Rows [cu[i], cu[i+1]) of q/out belong to sequence i (query j at position
 * j); its K/V are read through block_tables[seq_slot[i]] (max_blocks_per_seq entries per slot).
 *   q, out [q_rows, heads*head_dim] and the pools [pool_blocks, heads, 16, head_dim], all `dtype`.
 * bf16 with head_dim 64/128 runs on the tensor cores (tcgen05.mma, TMEM accumulators, TMA);
 * q must then be 16-byte aligned. Other shapes and f32 use the CUDA-core kernel. */
AK_API int ak_attn_prefill_paged(void* stream, const void* q, const void* k_pool, const void* v_pool,
                                 const int32_t* block_tables, uint32_t max_blocks_per_seq, const int32_t* cu,
                                 const int32_t* seq_slot, void* out, uint32_t n_seqs, uint32_t max_len,
                                 uint32_t q_rows, uint32_t heads, uint32_t head_dim, float scale, uint32_t dtype,
                                 uint32_t pool_blocks);

/* One kernel: h = x (+ residual, written back to x when given), y = rmsnorm(h) * w, then an
 * optional RoPE of y (adjacent pairs per head, positions[row]; head_dim = 0 disables).
 * y is f32 or bf16 (out_dtype). */
AK_API int ak_rmsnorm_rope_residual(void* stream, float* x, const float* residual, const float* w, void* y,
                                    const int32_t* positions, uint32_t rows, uint32_t size, float eps,
                                    uint32_t head_dim, uint32_t out_dtype);

/* bf16 tensor-core GEMM (tcgen05.mma, TMEM accumulator, TMA-staged operands):
 *   C[m,n] (op)= A[m,k] @ Wt[n,k]^T,  A bf16 row-major, Wt bf16 row-major (the TRANSPOSE of the
 *   reference's [k,n] weight, made once at upload), fp32 accumulate.
 * epilogue: see ak_gemm_epilogue. k must be a multiple of 8 (16-byte rows). */
typedef enum ak_gemm_epilogue {
    AK_EPI_STORE_F32 = 0,  /* C f32 = acc                     (matmul)            */
    AK_EPI_ADD_F32 = 1,    /* C f32 += acc                    (matmul_add)        */
    AK_EPI_STORE_BF16 = 2, /* C bf16 = acc                                        */
    AK_EPI_SILU_BF16 = 3   /* C bf16 = silu(acc)              (matmul + silu)     */
} ak_gemm_epilogue;
AK_API int ak_gemm_bf16(void* stream, const void* a, const void* wt, void* c, ak_matmul_meta m, uint32_t epilogue);
/* The same with an explicit row pitch of C, in elements (ldc >= n). The epilogue writes 16- and 32-byte vectors
 * when the pitch is a multiple of 8 elements and falls back to element stores otherwise, so an output with an odd
 * width (n = 50257, the lm_head) should be given a padded pitch (50264): the odd pitch costs ~7x in store time. */
AK_API int ak_gemm_bf16_ld(void* stream, const void* a, const void* wt, void* c, ak_matmul_meta m, uint32_t epilogue, uint32_t ldc);

/* Make the [n,k] bf16 operand from a reference-layout f32 [k,n] matrix (device to device). */
AK_API int ak_transpose_to_bf16(void* stream, const float* w_kn, void* wt_nk, uint32_t k, uint32_t n);
AK_API int ak_f32_to_bf16(void* stream, const float* src, void* dst, uint64_t n);
AK_API int ak_bf16_to_f32(void* stream, const void* src, float* dst, uint64_t n);

/* ================================================================== 2. session level */
typedef struct ak_ctx ak_ctx;         /* one device + one stream (Arc<B: Backend>) */
typedef struct ak_weights ak_weights; /* ModelWeights (src/nn/weights.rs:40-47)     */
typedef struct ak_session ak_session; /* InferenceSession (src/nn/inference.rs:13)  */

AK_API int ak_ctx_create(int device, ak_ctx** out); /* CudaBackend::new(device), src/main.rs:366 */
AK_API int ak_ctx_destroy(ak_ctx* ctx);
AK_API int ak_ctx_synchronize(ak_ctx* ctx);
AK_API void* ak_ctx_stream(ak_ctx* ctx);

/* Tensor parallelism (new: the reference runs on one device, src/main.rs:366). One process per
 * GPU; rank 0 makes an id with ak_tp_unique_id (128 bytes, ncclUniqueId), the host passes it to the
 * other ranks by its own means, and every rank calls ak_ctx_tp_init BEFORE creating weights.
 * Weights created on such a context hold this rank's slice (heads split over the fused qkv
 * columns and the out-proj rows, ffn columns / ffn-down rows); ak_weights_set_param still takes
 * the FULL tensor and keeps the slice. Sessions and engines then all-reduce (NCCL, sum, f32) the
 * partial out-proj and ffn-down products. All ranks must issue the same calls in the same order. */
AK_API int ak_tp_unique_id(void* out128);
AK_API int ak_ctx_tp_init(ak_ctx* ctx, uint32_t tp_size, uint32_t tp_rank, const void* unique_id128);
AK_API int ak_ctx_tp_shutdown(ak_ctx* ctx);

/* ModelWeights::zeros (src/nn/weights.rs:124-156): allocate all tensors, zero-filled. */
AK_API int ak_weights_create(ak_ctx* ctx, const ak_model_config* cfg, uint32_t dtype, ak_weights** out);
AK_API int ak_weights_destroy(ak_weights* w);
/* Number of tensors (1 + 6*layers + 2) and element count of tensor `index`, in
 * `ModelWeights::params()` order (src/nn/weights.rs:158-171): embedding, per block
 * {norm_1, qkv_proj, out_proj, norm_2, ffn_up, ffn_down}, final_norm, lm_head. */
AK_API uint32_t ak_weights_param_count(const ak_weights* w);
AK_API uint64_t ak_weights_param_len(const ak_weights* w, uint32_t index);
/* Tensor::copy_from_cpu per parameter (src/nn/checkpoint.rs:98-161 loads in this order).
 * `host` is f32 in the reference layout (matrices [in,out] row-major); the library converts to
 * its device layout (bf16 mode: cast, projection matrices stored transposed). */
AK_API int ak_weights_set_param(ak_weights* w, uint32_t index, const float* host, uint64_t n_elems);
/* Read a parameter back as f32 in the reference layout (bf16 mode returns the rounded values). */
AK_API int ak_weights_get_param(ak_weights* w, uint32_t index, float* host, uint64_t n_elems);
/* Fill every tensor on the device from a counter-based generator: matrices ~ N(0, std),
 * norm gains ~ N(1, std). Deterministic in (seed, index, element). For benchmarks. */
AK_API int ak_weights_init_synthetic(ak_weights* w, uint64_t seed, float std);

/* AKV3 checkpoints (src/nn/checkpoint.rs:18-36, 98-161): read the architecture header, and load
 * the weight tensors of a file into `w` (architecture and every tensor length are checked first,
 * as the reference's `load` does; the optimizer moments in the file are skipped). */
AK_API int ak_akv3_read_header(const char* path, ak_model_config* cfg_out, uint64_t* train_step_out);
AK_API int ak_weights_load_akv3(ak_weights* w, const char* path, uint64_t* train_step_out);

/* InferenceSession::new (src/nn/inference.rs:25-40). The cache is created with the session
 * but DETACHED, as in the reference (`cache: None`): prefill returns AK_NO_CACHE until
 * ak_session_attach_cache or ak_session_generate_greedy attaches it. */
AK_API int ak_session_create(ak_ctx* ctx, ak_weights* w, uint32_t max_context_len, ak_session** out);
AK_API int ak_session_destroy(ak_session* s);
/* replace_cache(Cache::new(..)) (src/nn/inference.rs:42-54): attach an empty cache. */
AK_API int ak_session_attach_cache(ak_session* s);
/* take_cache (src/nn/inference.rs:56-59): detach; the next prefill needs a new attach. */
AK_API int ak_session_take_cache(ak_session* s);
/* Cache::reset (src/nn/inference_graphs.rs:540-542): cur_len = 0, memory untouched. */
AK_API int ak_session_reset_cache(ak_session* s);
AK_API uint32_t ak_session_cur_len(const ak_session* s);
/* prefill (src/nn/inference.rs:61-176). logits_out: host f32[vocab] or NULL;
 * argmax_out: host uint32 or NULL (greedy token of the returned logits, computed on device). */
AK_API int ak_session_prefill(ak_session* s, const uint32_t* tokens, uint32_t n, float* logits_out, uint32_t* argmax_out);
/* decode_step (src/nn/inference.rs:178-262). */
AK_API int ak_session_decode_step(ak_session* s, uint32_t token, float* logits_out, uint32_t* argmax_out);
/* generate (src/nn/inference.rs:264-326) with temperature <= 0 and repetition_penalty == 1
 * (greedy, src/nn/sampling.rs:30-32): attaches a cache if none, prefill when the cache is empty
 * else decode_step over the prompt, then up to max_new tokens; stops after emitting `eos` when
 * stop_on_eos != 0, and stops quietly when the context fills. Token ids only cross PCIe. */
AK_API int ak_session_generate_greedy(ak_session* s, const uint32_t* prompt, uint32_t n, uint32_t max_new,
                                      int stop_on_eos, uint32_t* out_tokens, uint32_t* n_out);
/* generate (src/nn/inference.rs:264-326) with the reference's sampler on the device: every step's logits stay in
 * HBM, `sample_token` (src/nn/sampling.rs:18-81: repetition penalty over prompt + generated ids, temperature,
 * top-k, top-p, one uniform draw) runs as a kernel on them, and only the chosen id crosses PCIe. `run_chat` calls
 * it with (0.8, 40, 0.95, 1.15) (src/main.rs:160-162). temperature <= 0 is greedy over the penalised logits.
 * The draw of generated token t is the counter-based uniform number of (seed, t, row 0) that ak_sample_token
 * documents (the reference's generator is unseeded). top_k: 1..1024, or 0 = no truncation. */
AK_API int ak_session_generate(ak_session* s, const uint32_t* prompt, uint32_t n, uint32_t max_new, float temperature,
                               uint32_t top_k, float top_p, float repetition_penalty, uint64_t seed, int stop_on_eos,
                               uint32_t* out_tokens, uint32_t* n_out);
/* Copy the cached K (post-RoPE) and V rows 0..cur_len-1 of one layer to host as f32
 * [cur_len, dim] in the reference's contiguous layout (src/nn/inference_graphs.rs:511-543). */
AK_API int ak_session_read_cache(ak_session* s, uint32_t layer, float* k_out, float* v_out);

/* ================================================================== 3. engine level
 * Continuous batching: up to max_seqs sequences decode together, one launch per layer-op over
 * the ragged batch; a finished sequence's slot and KV blocks are reused by the next waiting one.
 * Block allocation is deterministic: lowest free block index first; a finished sequence's
 * blocks are returned before the next admission. */
typedef struct ak_engine ak_engine;
typedef struct ak_engine_config {
    uint32_t max_seqs;         /* concurrent sequences (64 in the headline config) */
    uint32_t max_seq_len;      /* longest prompt+generation of one sequence         */
    uint32_t kv_blocks;        /* KV pool size in blocks (0 = max_seqs * ceil(max_seq_len/16)) */
    uint32_t block_size;       /* must be 16 */
    uint32_t max_batch_tokens; /* token budget of one step (prefill + decode rows)  */
    uint32_t use_cuda_graph;   /* capture the decode-only step in a CUDA graph      */
    uint32_t stop_on_eos;      /* 0: run every sequence to its max_len              */
    uint32_t attn_timing;      /* record CUDA events around layer 0's decode attention */
    uint32_t async_steps;      /* 1: ak_engine_step returns once step N is LAUNCHED and step N-1's tokens are on the
                                * host, so describing and launching a step overlaps the previous step's GPU time.
                                * Needs stop_on_eos == 0 (sequence ends must be known without the tokens);
                                * ignored otherwise. poll / block_table / get_stats / clear_finished / run wait for
                                * the step in flight first. */
    uint32_t prefill_chunk_rows; /* Chunked prefill. 0 (default): every admitted prompt is prefilled whole, in the step that
                                  * admits it. N > 0: while other sequences are decoding, an admitted prompt is prefilled N rows
                                  * per step and its sequence samples its first token in the step that holds its last chunk; with
                                  * max_seqs + N <= 128 decode rows and prompt rows share ONE 128-row tile of every projection and
                                  * the prompt rides in the decode launches (no step is stretched by a long prompt). Needs bf16
                                  * weights, head_dim 64 or 128, no tensor parallelism; ignored otherwise. Tokens per sequence are
                                  * the same either way; admission times, hence block tables, differ. With nobody decoding, or more
                                  * than 8 chunks of prompt pending, prompts are prefilled whole. */
} ak_engine_config;

AK_API int ak_engine_create(ak_ctx* ctx, ak_weights* w, const ak_engine_config* cfg, ak_engine** out);
AK_API int ak_engine_destroy(ak_engine* e);
/* Queue a sequence: it generates until its total length reaches max_total_len (or eos). */
AK_API int ak_engine_submit(ak_engine* e, const uint32_t* prompt, uint32_t n, uint32_t max_total_len, uint64_t* seq_id);
/* One scheduler step: admit waiting sequences into free slots (their prompts are prefilled in
 * this step's ragged batch), run one token for every running sequence, retire finished ones.
 * n_running / n_finished_total may be NULL. Returns after the step's token ids are on the host. */
AK_API int ak_engine_step(ak_engine* e, uint32_t* n_running, uint32_t* n_waiting);
/* Steps until nothing is running or waiting (at most max_steps; 0 = no limit), then waits for the last
 * step. steps_done may be NULL. The loop the reference's `generate` runs per sequence
 * (src/nn/inference.rs:264-326), for the whole queue and without returning to the caller per token. */
AK_API int ak_engine_run(ak_engine* e, uint64_t max_steps, uint64_t* steps_done);
/* Has the sequence finished? Its generated tokens (prompt excluded) are copied to out (capacity
 * cap); n_out gets the count generated so far. */
AK_API int ak_engine_poll(ak_engine* e, uint64_t seq_id, uint32_t* out, uint32_t cap, uint32_t* n_out, int* finished);
/* Block table of a live or finished sequence (int32 block ids, in position order). */
AK_API int ak_engine_block_table(ak_engine* e, uint64_t seq_id, int32_t* out, uint32_t cap, uint32_t* n_out);
/* Forget finished sequences' records. */
AK_API int ak_engine_clear_finished(ak_engine* e);
typedef struct ak_engine_stats {
    uint64_t steps, decode_tokens, prefill_tokens, graph_launches, eager_steps, kernel_launches;
    double attn_ms_total;        /* sum of timed layer-0 decode-attention launches (attn_timing) */
    uint64_t attn_launches_timed;
    uint64_t attn_bytes_total;   /* algorithmic bytes of those launches */
    uint64_t h2d_bytes, d2h_bytes; /* bytes the engine copied host->device / device->host */
    double step_gpu_ms_total;      /* device time of the captured steps (attn_timing) */
    double launch_host_ms_total;   /* host time spent launching the captured steps */
    double decode_step_gpu_ms_total;  /* device time of the decode-only captured steps (attn_timing) */
    uint64_t decode_steps_timed;
    uint64_t decode_step_bytes_total; /* algorithmic bytes of those steps: every weight read once per step
                                       * (embedding rows of the batch only), K/V of all layers read for
                                       * every running sequence, one K/V position appended per sequence */
} ak_engine_stats;
AK_API int ak_engine_get_stats(ak_engine* e, ak_engine_stats* out);
AK_API int ak_engine_reset_stats(ak_engine* e);

#ifdef __cplusplus
}
#endif
#endif /* AKASHA_B200_H */
