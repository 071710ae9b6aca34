// Internal launcher interface between the kernels (*.cu) and the host runtime
// (runner / session / engine). All pointers are device pointers unless named *_host.
#pragma once
#include "common.cuh"

namespace ak {

// ---- elementwise.cu ----------------------------------------------------------------------
// Token source per row: tok_src[r] >= 0 is a literal id; tok_src[r] < 0 means "the token last
// sampled for sequence slot -(tok_src[r]+1)". Rows with slot_of_row[r] < 0 are zero-filled.
// idx_stride: distance (in int32) between consecutive rows' entries of tok_src / positions / slots.
int launch_embed_rows(cudaStream_t st, const int32_t* tok_src, uint32_t idx_stride, const uint32_t* sampled,
                      const void* table, uint32_t table_dtype, float* hidden, uint32_t vocab, uint32_t dim,
                      uint32_t rows);
// y[r] = rmsnorm(x[row_map ? row_map[r] : r]) * w ; rows whose mapped index is < 0 are zeroed.
int launch_rmsnorm(cudaStream_t st, const float* x, const float* w, void* y, uint32_t out_dtype,
                   const int32_t* row_map, uint32_t rows, uint32_t size, float eps);
int launch_rmsnorm_rope_residual(cudaStream_t st, float* x, const float* residual, const float* w, void* y,
                                 const int32_t* positions, uint32_t rows, uint32_t size, float eps,
                                 uint32_t head_dim, uint32_t out_dtype);
// qkv [T,3*dim] f32 -> q_out [T,dim] (q_dtype) with RoPE; K (RoPE) and V appended at slots[].
// rope_table: [max_pos][head_dim/2] float2 (cos,sin) or NULL (compute on device).
int launch_rope_kv_append(cudaStream_t st, const float* qkv, const int32_t* positions, const int32_t* slots,
                          uint32_t idx_stride, void* q_out, void* k_pool, void* v_pool, const float2* rope_table,
                          uint32_t rope_table_len, uint32_t tokens, uint32_t heads, uint32_t head_dim,
                          uint32_t block_size, uint32_t kv_dtype);
// Greedy argmax per row (first maximum wins). row_active: NULL or int32[rows]; rows with a
// negative entry keep their previous out_idx.
int launch_argmax(cudaStream_t st, const float* logits, uint32_t rows, uint32_t n, uint32_t ld,
                  const int32_t* row_active, uint32_t* out_idx);
int launch_silu(cudaStream_t st, float* x, uint64_t n);
// sample_token (src/nn/sampling.rs:18-81) per row; seen ids of row r are seen[seen_off[r] .. seen_off[r+1]).
int launch_sample_rows(cudaStream_t st, const float* logits, uint32_t rows, uint32_t n, uint32_t ld, const uint32_t* seen,
                       const uint32_t* seen_off, float penalty, float temperature, uint32_t top_k, float top_p, uint64_t seed,
                       uint64_t step, const int32_t* row_active, uint32_t* out_idx);
int launch_f32_to_bf16(cudaStream_t st, const float* src, void* dst, uint64_t n);
int launch_bf16_to_f32(cudaStream_t st, const void* src, float* dst, uint64_t n);
int launch_transpose_to_bf16(cudaStream_t st, const float* w_kn, void* wt_nk, uint32_t k, uint32_t n);
int launch_transpose_from_bf16(cudaStream_t st, const void* wt_nk, float* w_kn, uint32_t k, uint32_t n);
int launch_fill_normal(cudaStream_t st, void* dst, uint32_t dtype, uint64_t n, uint64_t seed, uint64_t stream_id,
                       float mean, float std);
// Matrix fill for (possibly sliced) weights: local element (i, c) of a [lin, lout] slice takes the
// value of the FULL matrix element it corresponds to, so every tensor-parallel rank and the
// single-GPU run hold the same model. col_mode 0: gc = col_off + c; 3: fused qkv blocks
// (gc = (c / blk_l) * blk_g + col_off + c % blk_l). transposed: storage is [lout, lin].
int launch_fill_normal_2d(cudaStream_t st, void* dst, uint32_t dtype, bool transposed, uint32_t lin, uint32_t lout,
                          uint32_t gout, uint32_t row_off, uint32_t col_mode, uint32_t col_off, uint32_t blk_l,
                          uint32_t blk_g, uint64_t seed, uint64_t stream_id, float mean, float std);
// Gather a sequence's paged rows back into the reference's contiguous [len, heads*head_dim] f32.
int launch_gather_paged(cudaStream_t st, const void* pool, uint32_t kv_dtype, const int32_t* block_table,
                        float* out, uint32_t len, uint32_t heads, uint32_t head_dim, uint32_t block_size);

// ---- gemm_simt.cu (true fp32) ---------------------------------------------------------------
enum { GEMM_ADD = 1, GEMM_SILU = 2 };
// C[m,n] (+)= A[m,k] @ B[k,n], row-major f32. m == 1 uses the cluster split-K GEMV.
int launch_gemm_f32(cudaStream_t st, const float* a, const float* b, float* c, uint32_t m, uint32_t n,
                    uint32_t k, uint32_t flags);

// ---- gemm_tcgen05.cu (bf16 tensor cores) --------------------------------------------------------
// invariant: keep the K summation structure a function of (n, k) only, so a row's result is the
// same whether 1 or 10,000 rows share the launch (the engine's batch invariance); costs some
// throughput for m > 128. false = fastest plan for the given m.
int launch_gemm_bf16(cudaStream_t st, const void* a, const void* wt, void* c, uint32_t m, uint32_t n,
                     uint32_t k, uint32_t epilogue, uint32_t ldc, bool invariant);
int gemm_bf16_check_status(cudaStream_t st);  // reads the device status word (syncs the stream)
// lm_head with the greedy argmax fused into the epilogue: every N tile writes each row's
// (max, first index) to part_val/part_idx [m][gemm_argmax_tiles()]; launch_argmax_finish reduces
// them (lowest index wins ties). logits may be NULL (nothing but the partials is written).
uint32_t gemm_argmax_tiles(uint32_t m, uint32_t n, uint32_t k);
int launch_gemm_bf16_argmax(cudaStream_t st, const void* a, const void* wt, float* logits, uint32_t ldc, float* part_val,
                            uint32_t* part_idx, uint32_t m, uint32_t n, uint32_t k);
int launch_argmax_finish(cudaStream_t st, const float* part_val, const uint32_t* part_idx, uint32_t rows, uint32_t tiles,
                         const int32_t* row_active, uint32_t* out_idx);

// ---- attn_decode.cu ----------------------------------------------------------------------------
size_t attn_decode_scratch_bytes(uint32_t rows, uint32_t heads, uint32_t head_dim, uint32_t n_splits);
uint32_t attn_decode_pick_splits(uint32_t rows, uint32_t heads, uint32_t head_dim, uint32_t kv_dtype, uint32_t max_kv_len);
// scratch (n_splits > 1): partials followed by one arrival counter per (row, head). The counters must be zero
// when the kernel starts and are zero again when it ends; counters_are_zero = false clears them on the stream first.
int launch_attn_decode_paged(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                             const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                             const ak_attn_decode_params& p, bool counters_are_zero);

// The same attention with the head split, RoPE and cache append of each sequence's new token done inside the kernel
// (replaces launch_rope_kv_append for rows that hold one decode token each): qkv [rows, 3*heads*head_dim] f32 is the
// qkv projection's output, position = kv_lens[row] - 1, slot = block_tables[row][pos/16]*16 + pos%16.
bool attn_decode_fused_supported(uint32_t head_dim);
// row_order (optional, int32[rows]): a permutation of the rows; CTAs are launched in that order (see attn_decode_row_order).
int launch_attn_decode_fused(cudaStream_t st, const float* qkv, const float2* rope_table, uint32_t rope_len, void* k_pool, void* v_pool,
                             const int32_t* block_tables, const int32_t* kv_lens, const int32_t* row_order, void* out, void* scratch,
                             const ak_attn_decode_params& p, bool counters_are_zero);
// Host side: the launch order that balances KV bytes over the SMs for these lengths (rows x heads CTAs of one launch).
void attn_decode_row_order(const int32_t* kv_lens, uint32_t rows, uint32_t heads, uint32_t head_dim, uint32_t kv_dtype, int32_t* order_out);
int attn_decode_status(unsigned int* out);  // device status word of the decode kernel
extern thread_local bool g_attn_early;      // true while the runner launches (cache untouched but for the newest positions)

}  // namespace ak
struct ak_ctx;
namespace ak {
// ---- tp.cu: in-place sum over the tensor-parallel group (no-op when tp_size == 1)
int tp_all_reduce_f32(ak_ctx* ctx, float* buf, size_t count);

// ---- attn_prefill.cu ---------------------------------------------------------------------------
// Causal varlen attention over newly prefilled sequences. q/out rows of sequence i are
// [cu[i], cu[i+1]) (+ row_base); K/V are read from the paged pools through the sequence's
// block table (block_tables[seq_slot[i]]). Query row j of a sequence sits at position pos0[i] + j and attends to
// positions 0 .. pos0[i] + j (pos0 == nullptr: all zero, a whole prompt; > 0: a later chunk of a prompt whose earlier
// positions are already cached). pos0 is honoured by the tensor-core kernel only (bf16, head_dim 64 / 128).
int launch_attn_prefill_paged(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                              const int32_t* block_tables, uint32_t max_blocks_per_seq, const int32_t* cu,
                              const int32_t* seq_slot, const int32_t* pos0, void* out, uint32_t n_seqs, uint32_t max_len,
                              uint32_t row_base, uint32_t heads, uint32_t head_dim, uint32_t block_size,
                              float scale, uint32_t dtype, uint64_t q_rows, uint64_t pool_blocks);
// ---- attn_prefill_tc.cu: the same contract on the tensor cores (bf16, head_dim 64/128). q has
// q_rows rows of heads*head_dim; the pools hold pool_blocks blocks. Waits that expire set a status word.
int launch_attn_prefill_tc(cudaStream_t st, const void* q, uint64_t q_rows, const void* k_pool, const void* v_pool,
                           uint64_t pool_blocks, const int32_t* block_tables, uint32_t max_blocks_per_seq, const int32_t* cu,
                           const int32_t* seq_slot, const int32_t* pos0, void* out, uint32_t n_seqs, uint32_t max_len, uint32_t row_base, uint32_t heads,
                           uint32_t head_dim, float scale);
int prefill_tc_status(unsigned int* out);
// The reference emitter's contiguous form (f32 q/k/v [*,dim], optional l_cache).
int launch_flash_attention_f32(cudaStream_t st, const float* q, const float* k, const float* v, float* out,
                               float* l_cache, ak_flash_attn_meta m);

}  // namespace ak
