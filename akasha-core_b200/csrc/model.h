// Host runtime shared by the session and engine levels of the C ABI: context, weights in the
// `ModelWeights::params()` order, and the ragged-batch runner that launches one kernel per
// layer-op over all token rows of a step.
#pragma once
#include <map>
#include <vector>

#include "kernels.h"

struct ak_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    // tensor parallelism (1 = off): this context is rank tp_rank of tp_size, tp_comm = ncclComm_t
    uint32_t tp_size = 1, tp_rank = 0;
    void* tp_comm = nullptr;
};

struct ak_weights {
    ak_ctx* ctx = nullptr;
    ak_model_config cfg{};
    uint32_t dtype = AK_F32;
    // Device tensors. f32 mode: matrices f32 [in,out] (the reference layout, src/nn/weights.rs:32-47).
    // bf16 mode: embedding bf16 [vocab,dim]; projection matrices bf16 [out,in] (transposed once at
    // upload so both tcgen05 operands are K-major); norm gains stay f32.
    void* embedding = nullptr;
    struct Block {
        float* norm_1 = nullptr;
        void* qkv = nullptr;
        void* out = nullptr;
        float* norm_2 = nullptr;
        void* up = nullptr;
        void* down = nullptr;
    };
    std::vector<Block> blocks;
    float* final_norm = nullptr;
    void* lm_head = nullptr;
    float* staging = nullptr;  // f32 staging for layout conversion
    size_t staging_elems = 0;

    struct ParamRef {
        void** ptr;
        uint64_t len;
        uint32_t kind;  // 0 = norm gain (f32), 1 = embedding table, 2 = matrix [in,out]
        uint32_t in, out;    // full (reference) shape
        // tensor-parallel slice held by this rank: 0 = whole tensor, 1 = rows (in) split,
        // 2 = columns (out) split, 3 = the fused qkv matrix: each of its q|k|v column blocks split
        uint32_t split = 0;
        uint32_t lin = 0, lout = 0;  // local shape
        uint64_t llen = 0;           // local element count
    };
    uint32_t tp_size = 1, tp_rank = 0;
    std::vector<ParamRef> params;  // params() order
};

namespace ak {

// One int4 per token row of a step.
struct RowInfo {
    int32_t tok_src;  // >= 0 literal id; < 0: -(slot+1) = last sampled token of that slot; INT32_MIN inactive
    int32_t pos;      // position in its sequence, -1 inactive
    int32_t slot;     // paged KV slot for the append, -1 none
    int32_t seq;      // sequence slot the row belongs to
};

struct StepDesc {  // offsets (in int32 units) into the descriptor buffer
    uint32_t kv_lens, out_rows, row_order, pf_cu, pf_slot, pf_pos0, block_tables, rows, total;
};

class Runner {
   public:
    Runner() = default;
    ~Runner();
    int init(ak_ctx* ctx, ak_weights* w, uint32_t max_seqs, uint32_t max_seq_len, uint32_t kv_blocks, uint32_t max_prefill_tokens);
    // Host mirror of the descriptor (pinned). Fill, then run().
    int32_t* h_kv_lens() { return h_desc_ + d_.kv_lens; }
    int32_t* h_out_rows() { return h_desc_ + d_.out_rows; }
    int32_t* h_row_order() { return h_desc_ + d_.row_order; }   // launch order of the decode attention's rows (filled by run*)
    int32_t* h_pf_cu() { return h_desc_ + d_.pf_cu; }
    int32_t* h_pf_slot() { return h_desc_ + d_.pf_slot; }
    // position of the first prompt row of every prefilled sequence of the step: 0 for a whole prompt, the number of
    // tokens already cached when the prompt is prefilled in chunks over several steps
    int32_t* h_pf_pos0() { return h_desc_ + d_.pf_pos0; }
    // chunked prefill needs the tensor-core prefill kernel, which takes the chunk's first position (bf16, head_dim 64/128)
    bool chunked_prefill_supported() const;
    int32_t* h_block_table(uint32_t seq) { return h_desc_ + d_.block_tables + (size_t)seq * max_blocks_; }
    RowInfo* h_rows() { return reinterpret_cast<RowInfo*>(h_desc_ + d_.rows); }
    const uint32_t* h_sampled() const { return h_sampled_; }

    // Launch one step over rows [0, max_seqs_) (decode rows, one per slot) plus n_prefill_rows
    // prefill rows. Ends with the sampled tokens copied to the pinned host buffer (async).
    int run(uint32_t n_prefill_rows, uint32_t n_pf_seqs, uint32_t max_pf_len, bool any_decode, uint32_t max_kv_len);
    // Decode-only step through a captured CUDA graph (captured on first use).
    int run_decode_graph(uint32_t max_kv_len_hint);
    // Any step (decode rows + optional prefill rows) through a per-bucket captured graph.
    int run_graph(uint32_t n_prefill_rows, uint32_t n_pf_seqs, uint32_t max_pf_len);
    int sync();
    // Two banks of host-side step state (pinned descriptor, pinned result buffer, timing events, captured
    // graphs), so that the host can describe and launch step N+1 while step N is still running. The
    // accessors above and run()/run_graph() use the current bank; the device buffers are shared and
    // ordered by the stream.
    void set_bank(uint32_t b);
    uint32_t bank() const { return bank_; }
    int mark_done();               // record "the step launched from the current bank is complete"
    int wait_bank(uint32_t b);     // block until the step last launched from bank b is complete
    int read_logits(uint32_t slot, float* host_out);
    int gather_cache(uint32_t layer, const int32_t* h_table, uint32_t len, float* k_out, float* v_out);

    const float* logits_dev() const { return logits_; }     // [max_seqs][logits_ld()] f32, written when keep_logits
    uint32_t logits_ld() const { return logits_ld_; }
    uint32_t* sampled_dev() { return d_sampled_; }           // the token every slot feeds to its next decode row
    uint32_t max_seqs() const { return max_seqs_; }
    uint32_t max_blocks() const { return max_blocks_; }
    uint32_t n_blocks() const { return n_blocks_; }
    uint32_t max_prefill_tokens() const { return max_pf_tokens_; }
    uint32_t dtype() const { return w_->dtype; }
    uint32_t local_qdim() const { return dq_; }  // heads held by this rank x head_dim
    void enable_attn_timing(bool on) { attn_timing_ = on; }
    void set_keep_logits(bool on) { keep_logits_ = on; }
    float last_attn_ms();
    float last_step_gpu_ms();          // device time of the last captured step (attn timing on)
    double launch_host_ms = 0.0;       // host time spent inside cudaGraphLaunch, accumulated
    uint64_t graph_launches = 0, eager_steps = 0;
    uint64_t h2d_bytes = 0, d2h_bytes = 0;   // bytes copied by run() / run_decode_graph()
    uint64_t graph_kernels = 0;              // kernel launches recorded in the captured decode step

   private:
    int launch_layers(uint32_t T, uint32_t n_pf_rows, uint32_t n_pf_seqs, uint32_t max_pf_len, bool any_decode, uint32_t n_splits, bool capturing);
    int gemm(const void* a, const void* w, void* c, uint32_t m, uint32_t n, uint32_t k, int mode);

    ak_ctx* ctx_ = nullptr;
    ak_weights* w_ = nullptr;
    uint32_t max_seqs_ = 0, max_blocks_ = 0, n_blocks_ = 0, max_pf_tokens_ = 0, max_rows_ = 0, max_seq_len_ = 0;
    StepDesc d_{};
    int32_t* h_desc_ = nullptr;  // pinned
    int32_t* d_desc_ = nullptr;
    uint32_t* h_sampled_ = nullptr;  // pinned
    uint32_t* d_sampled_ = nullptr;
    std::vector<void*> k_pool_, v_pool_;
    float* hidden_ = nullptr;
    void* xn_ = nullptr;
    float* qkv_ = nullptr;
    void* qbuf_ = nullptr;
    void* attn_ = nullptr;
    void* up_ = nullptr;
    void* xf_ = nullptr;
    float* logits_ = nullptr;
    uint32_t logits_ld_ = 0;          // row pitch of logits_ (padded to 4 in bf16 mode)
    bool keep_logits_ = true;         // false: the engine never reads logits, only the argmax
    float* amax_val_ = nullptr;       // per-tile row maxima of the lm_head (bf16 mode)
    uint32_t* amax_idx_ = nullptr;
    uint32_t amax_tiles_ = 0;
    float* tp_tmp_ = nullptr;         // [rows, dim] f32 partial of the row-split projections (tp > 1)
    uint32_t tp_ = 1, heads_l_ = 0, dq_ = 0, ffn_l_ = 0;  // local heads, local q width, local ffn width
    float* attn_scratch_ = nullptr;
    size_t attn_scratch_bytes_ = 0;
    float2* rope_table_ = nullptr;
    uint32_t rope_len_ = 0;
    struct StepGraph {
        cudaGraphExec_t exec = nullptr;
        uint64_t kernels = 0;
        size_t h2d = 0;
    };
    std::map<uint64_t, StepGraph> graphs_;  // key = (prefill row bucket << 32) | prefill sequence bucket
    bool attn_timing_ = false;
    cudaEvent_t ev_attn0_ = nullptr, ev_attn1_ = nullptr, ev_g0_ = nullptr, ev_g1_ = nullptr;
    bool ev_g_valid_ = false;
    // AK_TRACE=1 (eager steps only): one event after every launch, per-launch times to stderr
    std::vector<cudaEvent_t> trace_ev_;
    std::vector<const char*> trace_lbl_;
    size_t trace_n_ = 0;
    std::vector<cudaEvent_t> gtrace_ev_;      // the same inside the captured decode step (event-record nodes)
    std::vector<const char*> gtrace_lbl_;
    bool gtrace_capture_ = false, gtrace_ran_ = false;
    void trace_mark(const char* label);
    void trace_dump();
    bool ev_valid_ = false;
    struct Bank {
        int32_t* h_desc = nullptr;
        uint32_t* h_sampled = nullptr;
        cudaEvent_t ev_attn0 = nullptr, ev_attn1 = nullptr, ev_g0 = nullptr, ev_g1 = nullptr, ev_done = nullptr;
        bool ev_valid = false, ev_g_valid = false;
    } banks_[2];
    uint32_t bank_ = 0;
    // Admission steps: the admitted prompts' rows run on a second stream, concurrently with the decode
    // rows (different sequences: they share nothing until the final norm).
    cudaStream_t st2_ = nullptr;
    cudaEvent_t ev_fork_ = nullptr, ev_join_ = nullptr;
    cudaStream_t st_time_ = nullptr;                       // side stream the attention timestamps are taken on
    cudaEvent_t ev_tfork_ = nullptr, ev_tjoin_ = nullptr;
    bool time_forked_ = false;
    int attn_time_mark(cudaStream_t s, cudaEvent_t ev, bool capturing);
    bool two_streams_ = true;
};

}  // namespace ak
