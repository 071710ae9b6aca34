// Context, weights (ModelWeights layout, src/nn/weights.rs:32-171) and the ragged-batch runner.
#include "model.h"

#include <math.h>
#include <limits.h>
#include <string.h>

#include <stdlib.h>

#include <chrono>

using namespace ak;

// ======================================================================== context
extern "C" {

int ak_ctx_create(int device, ak_ctx** out) {
    AK_REQUIRE(out, AK_ERR_INVALID_ARG, "ak_ctx_create: null pointer");
    int n = 0;
    AK_CUDA(cudaGetDeviceCount(&n));
    AK_REQUIRE(device >= 0 && device < n, AK_ERR_INVALID_ARG, "ak_ctx_create: device %d out of range (%d present)", device, n);
    AK_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    AK_CUDA(cudaGetDeviceProperties(&prop, device));
    AK_REQUIRE(prop.major == 10, AK_ERR_UNSUPPORTED,
               "ak_ctx_create: device %d is sm_%d%d; this library is built for sm_100a (B200) only", device, prop.major, prop.minor);
    ak_ctx* c = new ak_ctx();
    c->device = device;
    AK_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    *out = c;
    return AK_OK;
}
int ak_ctx_tp_shutdown(ak_ctx* ctx);
int ak_ctx_destroy(ak_ctx* ctx) {
    if (!ctx) return AK_OK;
    cudaSetDevice(ctx->device);
    ak_ctx_tp_shutdown(ctx);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return AK_OK;
}
int ak_ctx_synchronize(ak_ctx* ctx) {
    AK_REQUIRE(ctx, AK_ERR_INVALID_ARG, "ak_ctx_synchronize: null ctx");
    AK_CUDA(cudaStreamSynchronize(ctx->stream));
    return AK_OK;
}
void* ak_ctx_stream(ak_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

// ======================================================================== weights
static size_t welem(uint32_t dtype) { return dtype == AK_F32 ? 4 : 2; }

int ak_weights_create(ak_ctx* ctx, const ak_model_config* cfg, uint32_t dtype, ak_weights** out) {
    AK_REQUIRE(ctx && cfg && out, AK_ERR_INVALID_ARG, "ak_weights_create: null pointer");
    AK_REQUIRE(dtype <= AK_BF16, AK_ERR_INVALID_ARG, "ak_weights_create: bad dtype %u", dtype);
    AK_REQUIRE(cfg->num_layers >= 1 && cfg->num_heads >= 1 && cfg->dim % cfg->num_heads == 0 && cfg->vocab_size >= 1 && cfg->ffn_hidden >= 1,
               AK_ERR_INVALID_ARG, "ak_weights_create: bad config (layers >= 1, dim %% heads == 0 required)");
    const uint32_t hd = cfg->dim / cfg->num_heads;
    AK_REQUIRE(hd % 2 == 0, AK_ERR_INVALID_ARG, "ak_weights_create: head_dim must be even (RoPE pairs)");
    if (dtype == AK_BF16)
        AK_REQUIRE(cfg->dim % 8 == 0 && cfg->ffn_hidden % 8 == 0 && hd % 8 == 0, AK_ERR_UNSUPPORTED,
                   "ak_weights_create: bf16 mode needs dim, ffn_hidden and head_dim to be multiples of 8");
    else
        AK_REQUIRE(hd % 4 == 0, AK_ERR_UNSUPPORTED, "ak_weights_create: head_dim must be a multiple of 4");
    const uint32_t tp = ctx->tp_size;
    AK_REQUIRE(cfg->num_heads % tp == 0 && cfg->ffn_hidden % tp == 0, AK_ERR_INVALID_ARG,
               "ak_weights_create: heads and ffn_hidden must be divisible by the tensor-parallel size %u", tp);
    if (dtype == AK_BF16) AK_REQUIRE((cfg->ffn_hidden / tp) % 8 == 0, AK_ERR_UNSUPPORTED, "ak_weights_create: ffn_hidden / tp must be a multiple of 8");
    AK_CUDA(cudaSetDevice(ctx->device));
    ak_weights* w = new ak_weights();
    w->ctx = ctx;
    w->cfg = *cfg;
    w->dtype = dtype;
    w->tp_size = tp;
    w->tp_rank = ctx->tp_rank;
    const uint64_t V = cfg->vocab_size, D = cfg->dim, F = cfg->ffn_hidden;
    const uint32_t Dl = (uint32_t)D / tp, Fl = (uint32_t)F / tp;
    w->blocks.resize(cfg->num_layers);
    // split: 0 whole, 1 rows, 2 columns, 3 fused-qkv columns (only when tp > 1)
    auto add = [&](void** p, uint64_t len, uint32_t kind, uint32_t in, uint32_t o, uint32_t split) {
        ak_weights::ParamRef pr{};
        pr.ptr = p; pr.len = len; pr.kind = kind; pr.in = in; pr.out = o;
        pr.split = tp > 1 ? split : 0;
        pr.lin = in; pr.lout = o;
        if (pr.split == 1) pr.lin = in / tp;
        if (pr.split == 2) pr.lout = o / tp;
        if (pr.split == 3) pr.lout = 3 * Dl;
        pr.llen = kind == 0 ? len : (uint64_t)pr.lin * pr.lout;
        w->params.push_back(pr);
    };
    (void)Fl;
    add(&w->embedding, V * D, 1, (uint32_t)V, (uint32_t)D, 0);
    for (auto& b : w->blocks) {
        add((void**)&b.norm_1, D, 0, 0, 0, 0);
        add(&b.qkv, D * 3 * D, 2, (uint32_t)D, (uint32_t)(3 * D), 3);  // heads split: columns of q, k and v
        add(&b.out, D * D, 2, (uint32_t)D, (uint32_t)D, 1);            // rows follow the local heads
        add((void**)&b.norm_2, D, 0, 0, 0, 0);
        add(&b.up, D * F, 2, (uint32_t)D, (uint32_t)F, 2);
        add(&b.down, F * D, 2, (uint32_t)F, (uint32_t)D, 1);
    }
    add((void**)&w->final_norm, D, 0, 0, 0, 0);
    add(&w->lm_head, D * V, 2, (uint32_t)D, (uint32_t)V, 0);
    for (auto& pr : w->params) {
        size_t bytes = pr.llen * (pr.kind == 0 ? 4 : welem(dtype));
        cudaError_t e = cudaMalloc(pr.ptr, bytes);
        if (e != cudaSuccess) {
            ak_weights_destroy(w);
            return cuda_fail(e, "cudaMalloc(weights)", __FILE__, __LINE__);
        }
        cudaMemsetAsync(*pr.ptr, 0, bytes, ctx->stream);
    }
    AK_CUDA(cudaStreamSynchronize(ctx->stream));
    *out = w;
    return AK_OK;
}

int ak_weights_destroy(ak_weights* w) {
    if (!w) return AK_OK;
    cudaSetDevice(w->ctx->device);
    for (auto& pr : w->params)
        if (*pr.ptr) cudaFree(*pr.ptr);
    if (w->staging) cudaFree(w->staging);
    delete w;
    return AK_OK;
}

uint32_t ak_weights_param_count(const ak_weights* w) { return w ? (uint32_t)w->params.size() : 0; }
uint64_t ak_weights_param_len(const ak_weights* w, uint32_t index) {
    return (w && index < w->params.size()) ? w->params[index].len : 0;
}

static int ensure_staging(ak_weights* w, size_t elems) {
    if (w->staging_elems >= elems) return AK_OK;
    if (w->staging) cudaFree(w->staging);
    w->staging = nullptr;
    w->staging_elems = 0;
    AK_CUDA(cudaMalloc((void**)&w->staging, elems * sizeof(float)));
    w->staging_elems = elems;
    return AK_OK;
}

int ak_weights_set_param(ak_weights* w, uint32_t index, const float* host, uint64_t n_elems) {
    AK_REQUIRE(w && host, AK_ERR_INVALID_ARG, "ak_weights_set_param: null pointer");
    AK_REQUIRE(index < w->params.size(), AK_ERR_INVALID_ARG, "ak_weights_set_param: index %u out of range", index);
    auto& pr = w->params[index];
    AK_REQUIRE(n_elems == pr.len, AK_ERR_INVALID_ARG, "ak_weights_set_param: tensor %u holds %llu elements, got %llu", index,
               (unsigned long long)pr.len, (unsigned long long)n_elems);
    AK_CUDA(cudaSetDevice(w->ctx->device));
    cudaStream_t st = w->ctx->stream;
    // tensor-parallel slice of the full host tensor (the caller always passes the whole tensor)
    std::vector<float> slice;
    const float* src = host;
    if (pr.split == 1) {
        src = host + (size_t)w->tp_rank * pr.lin * pr.out;  // contiguous block of rows
    } else if (pr.split == 2 || pr.split == 3) {
        slice.resize(pr.llen);
        const uint32_t nblk = pr.split == 3 ? 3 : 1;
        const uint32_t bl = pr.lout / nblk, bg = pr.out / nblk;  // local / global block width
        for (uint32_t i = 0; i < pr.lin; i++)
            for (uint32_t b = 0; b < nblk; b++)
                memcpy(&slice[(size_t)i * pr.lout + (size_t)b * bl], host + (size_t)i * pr.out + (size_t)b * bg + (size_t)w->tp_rank * bl, (size_t)bl * 4);
        src = slice.data();
    }
    if (w->dtype == AK_F32 || pr.kind == 0) {
        AK_CUDA(cudaMemcpyAsync(*pr.ptr, src, pr.llen * 4, cudaMemcpyHostToDevice, st));
    } else {
        int rc = ensure_staging(w, pr.llen);
        if (rc) return rc;
        AK_CUDA(cudaMemcpyAsync(w->staging, src, pr.llen * 4, cudaMemcpyHostToDevice, st));
        rc = (pr.kind == 1) ? launch_f32_to_bf16(st, w->staging, *pr.ptr, pr.llen)
                            : launch_transpose_to_bf16(st, w->staging, *pr.ptr, pr.lin, pr.lout);
        if (rc) return rc;
    }
    AK_CUDA(cudaStreamSynchronize(st));
    return AK_OK;
}

int ak_weights_get_param(ak_weights* w, uint32_t index, float* host, uint64_t n_elems) {
    AK_REQUIRE(w && host, AK_ERR_INVALID_ARG, "ak_weights_get_param: null pointer");
    AK_REQUIRE(index < w->params.size(), AK_ERR_INVALID_ARG, "ak_weights_get_param: index %u out of range", index);
    auto& pr = w->params[index];
    AK_REQUIRE(n_elems == pr.len, AK_ERR_INVALID_ARG, "ak_weights_get_param: tensor %u holds %llu elements", index, (unsigned long long)pr.len);
    AK_REQUIRE(pr.split == 0, AK_ERR_UNSUPPORTED, "ak_weights_get_param: tensor %u is sliced across tensor-parallel ranks", index);
    AK_CUDA(cudaSetDevice(w->ctx->device));
    cudaStream_t st = w->ctx->stream;
    if (w->dtype == AK_F32 || pr.kind == 0) {
        AK_CUDA(cudaMemcpyAsync(host, *pr.ptr, pr.len * 4, cudaMemcpyDeviceToHost, st));
    } else {
        int rc = ensure_staging(w, pr.len);
        if (rc) return rc;
        rc = (pr.kind == 1) ? launch_bf16_to_f32(st, *pr.ptr, w->staging, pr.len)
                            : launch_transpose_from_bf16(st, *pr.ptr, w->staging, pr.in, pr.out);
        if (rc) return rc;
        AK_CUDA(cudaMemcpyAsync(host, w->staging, pr.len * 4, cudaMemcpyDeviceToHost, st));
    }
    AK_CUDA(cudaStreamSynchronize(st));
    return AK_OK;
}

int ak_weights_init_synthetic(ak_weights* w, uint64_t seed, float std) {
    AK_REQUIRE(w, AK_ERR_INVALID_ARG, "ak_weights_init_synthetic: null pointer");
    AK_CUDA(cudaSetDevice(w->ctx->device));
    for (size_t i = 0; i < w->params.size(); i++) {
        auto& pr = w->params[i];
        int rc;
        if (pr.kind == 2) {
            const uint32_t nblk = pr.split == 3 ? 3 : 1;
            const uint32_t bl = pr.lout / nblk, bg = pr.out / nblk;
            rc = launch_fill_normal_2d(w->ctx->stream, *pr.ptr, w->dtype, w->dtype == AK_BF16, pr.lin, pr.lout, pr.out,
                                       pr.split == 1 ? w->tp_rank * pr.lin : 0, pr.split == 3 ? 3 : 0,
                                       (pr.split == 2 || pr.split == 3) ? w->tp_rank * bl : 0, bl, bg, seed, i, 0.0f, std);
        } else {
            rc = launch_fill_normal(w->ctx->stream, *pr.ptr, pr.kind == 0 ? (uint32_t)AK_F32 : w->dtype, pr.len, seed, i,
                                    pr.kind == 0 ? 1.0f : 0.0f, std);
        }
        if (rc) return rc;
    }
    AK_CUDA(cudaStreamSynchronize(w->ctx->stream));
    return AK_OK;
}

}  // extern "C"

// ======================================================================== runner
namespace ak {

static uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

Runner::~Runner() {
    if (!ctx_) return;
    cudaSetDevice(ctx_->device);
    cudaStreamSynchronize(ctx_->stream);
    if (st2_) cudaStreamSynchronize(st2_);
    if (st_time_) cudaStreamSynchronize(st_time_);
    for (auto& kv : graphs_) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    if (ev_fork_) cudaEventDestroy(ev_fork_);
    if (ev_join_) cudaEventDestroy(ev_join_);
    if (st2_) cudaStreamDestroy(st2_);
    if (ev_tfork_) cudaEventDestroy(ev_tfork_);
    if (ev_tjoin_) cudaEventDestroy(ev_tjoin_);
    if (st_time_) cudaStreamDestroy(st_time_);
    for (Bank& b : banks_) {
        if (b.ev_attn0) cudaEventDestroy(b.ev_attn0);
        if (b.ev_attn1) cudaEventDestroy(b.ev_attn1);
        if (b.ev_g0) cudaEventDestroy(b.ev_g0);
        if (b.ev_g1) cudaEventDestroy(b.ev_g1);
        if (b.ev_done) cudaEventDestroy(b.ev_done);
    }
    for (void* p : k_pool_) cudaFree(p);
    for (void* p : v_pool_) cudaFree(p);
    cudaFree(hidden_); cudaFree(xn_); cudaFree(qkv_); cudaFree(qbuf_); cudaFree(attn_); cudaFree(up_);
    cudaFree(amax_val_); cudaFree(amax_idx_); cudaFree(tp_tmp_);
    cudaFree(xf_); cudaFree(logits_); cudaFree(attn_scratch_); cudaFree(rope_table_);
    cudaFree(d_desc_); cudaFree(d_sampled_);
    for (Bank& b : banks_) {
        if (b.h_desc) cudaFreeHost(b.h_desc);
        if (b.h_sampled) cudaFreeHost(b.h_sampled);
    }
}

int Runner::init(ak_ctx* ctx, ak_weights* w, uint32_t max_seqs, uint32_t max_seq_len, uint32_t kv_blocks, uint32_t max_prefill_tokens) {
    ctx_ = ctx;
    w_ = w;
    AK_CUDA(cudaSetDevice(ctx->device));
    const ak_model_config& c = w->cfg;
    const uint32_t D = c.dim, F = c.ffn_hidden, V = c.vocab_size, H = c.num_heads, hd = D / H;
    max_seqs_ = max_seqs;
    max_seq_len_ = max_seq_len;
    max_blocks_ = (max_seq_len + 15) / 16;
    n_blocks_ = kv_blocks ? kv_blocks : max_seqs * max_blocks_;
    max_pf_tokens_ = max_prefill_tokens;
    max_rows_ = max_seqs + max_prefill_tokens;
    const size_t act = welem(w->dtype);
    AK_REQUIRE(w->tp_size == ctx->tp_size && w->tp_rank == ctx->tp_rank, AK_ERR_INVALID_ARG, "runner: weights and context disagree on the tensor-parallel layout");
    tp_ = w->tp_size;
    heads_l_ = H / tp_;
    dq_ = heads_l_ * hd;
    ffn_l_ = F / tp_;

    d_.kv_lens = 0;
    d_.out_rows = d_.kv_lens + max_seqs;
    d_.row_order = d_.out_rows + max_seqs;
    d_.pf_cu = d_.row_order + max_seqs;
    d_.pf_slot = d_.pf_cu + max_seqs + 1;
    d_.pf_pos0 = d_.pf_slot + max_seqs;
    d_.block_tables = d_.pf_pos0 + max_seqs;
    d_.rows = align_up(d_.block_tables + max_seqs * max_blocks_, 4);
    d_.total = d_.rows + max_rows_ * 4;
    for (Bank& b : banks_) {
        AK_CUDA(cudaMallocHost((void**)&b.h_desc, (size_t)d_.total * 4));
        memset(b.h_desc, 0, (size_t)d_.total * 4);
        AK_CUDA(cudaMallocHost((void**)&b.h_sampled, (size_t)max_seqs * 4));
        memset(b.h_sampled, 0, (size_t)max_seqs * 4);
    }
    bank_ = 0;
    h_desc_ = banks_[0].h_desc;
    h_sampled_ = banks_[0].h_sampled;
    AK_CUDA(cudaMalloc((void**)&d_desc_, (size_t)d_.total * 4));
    AK_CUDA(cudaMemset(d_desc_, 0, (size_t)d_.total * 4));

    AK_CUDA(cudaMalloc((void**)&d_sampled_, (size_t)max_seqs * 4));
    AK_CUDA(cudaMemset(d_sampled_, 0, (size_t)max_seqs * 4));

    const size_t pool_bytes = (size_t)n_blocks_ * heads_l_ * 16 * hd * act;  // each rank caches its own heads
    k_pool_.assign(c.num_layers, nullptr);
    v_pool_.assign(c.num_layers, nullptr);
    for (uint32_t l = 0; l < c.num_layers; l++) {
        AK_CUDA(cudaMalloc(&k_pool_[l], pool_bytes));
        AK_CUDA(cudaMalloc(&v_pool_[l], pool_bytes));
        AK_CUDA(cudaMemsetAsync(k_pool_[l], 0, pool_bytes, ctx->stream));
        AK_CUDA(cudaMemsetAsync(v_pool_[l], 0, pool_bytes, ctx->stream));
    }
    const size_t R = max_rows_;
    AK_CUDA(cudaMalloc((void**)&hidden_, R * D * 4));
    AK_CUDA(cudaMalloc(&xn_, R * D * act));
    AK_CUDA(cudaMalloc((void**)&qkv_, R * 3 * dq_ * 4));
    AK_CUDA(cudaMalloc(&qbuf_, R * dq_ * act));
    AK_CUDA(cudaMalloc(&attn_, R * dq_ * act));
    AK_CUDA(cudaMalloc(&up_, R * ffn_l_ * act));
    if (tp_ > 1) {
        AK_CUDA(cudaMalloc((void**)&tp_tmp_, R * D * 4));
        AK_CUDA(cudaMemsetAsync(tp_tmp_, 0, R * D * 4, ctx->stream));
    }
    AK_CUDA(cudaMalloc(&xf_, (size_t)max_seqs * D * act));
    logits_ld_ = (w->dtype == AK_BF16) ? (V + 3) / 4 * 4 : V;
    AK_CUDA(cudaMalloc((void**)&logits_, (size_t)max_seqs * logits_ld_ * 4));
    if (w->dtype == AK_BF16) {
        amax_tiles_ = gemm_argmax_tiles(max_seqs, V, D);
        AK_CUDA(cudaMalloc((void**)&amax_val_, (size_t)max_seqs * amax_tiles_ * 4));
        AK_CUDA(cudaMalloc((void**)&amax_idx_, (size_t)max_seqs * amax_tiles_ * 4));
    }
    AK_CUDA(cudaMemsetAsync(hidden_, 0, R * D * 4, ctx->stream));
    AK_CUDA(cudaMemsetAsync(xn_, 0, R * D * act, ctx->stream));
    AK_CUDA(cudaMemsetAsync(qkv_, 0, R * 3 * dq_ * 4, ctx->stream));
    AK_CUDA(cudaMemsetAsync(qbuf_, 0, R * dq_ * act, ctx->stream));
    AK_CUDA(cudaMemsetAsync(attn_, 0, R * dq_ * act, ctx->stream));
    AK_CUDA(cudaMemsetAsync(up_, 0, R * ffn_l_ * act, ctx->stream));
    AK_CUDA(cudaMemsetAsync(logits_, 0, (size_t)max_seqs * logits_ld_ * 4, ctx->stream));
    attn_scratch_bytes_ = attn_decode_scratch_bytes(max_seqs, heads_l_, hd, 32);
    AK_CUDA(cudaMalloc((void**)&attn_scratch_, attn_scratch_bytes_));
    AK_CUDA(cudaMemsetAsync(attn_scratch_, 0, attn_scratch_bytes_, ctx->stream));   // arrival counters start at zero

    // RoPE factors from the host libm, exactly as the reference's CPU kernel forms them
    // (src/shaders/cpu.rs:98-100): freq = 1/powf(10000, d/hd), angle = (float)pos * freq.
    rope_len_ = max_seq_len;
    std::vector<float2> tab((size_t)rope_len_ * (hd / 2));
    for (uint32_t pos = 0; pos < rope_len_; pos++)
        for (uint32_t d = 0; d < hd; d += 2) {
            float freq = 1.0f / powf(10000.0f, (float)d / (float)hd);
            float angle = (float)pos * freq;
            tab[(size_t)pos * (hd / 2) + d / 2] = make_float2(cosf(angle), sinf(angle));
        }
    AK_CUDA(cudaMalloc((void**)&rope_table_, tab.size() * sizeof(float2)));
    AK_CUDA(cudaMemcpyAsync(rope_table_, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice, ctx->stream));
    for (Bank& b : banks_) {
        AK_CUDA(cudaEventCreate(&b.ev_attn0));
        AK_CUDA(cudaEventCreate(&b.ev_attn1));
        AK_CUDA(cudaEventCreate(&b.ev_g0));
        AK_CUDA(cudaEventCreate(&b.ev_g1));
        AK_CUDA(cudaEventCreateWithFlags(&b.ev_done, cudaEventDisableTiming));
    }
    ev_attn0_ = banks_[0].ev_attn0; ev_attn1_ = banks_[0].ev_attn1; ev_g0_ = banks_[0].ev_g0; ev_g1_ = banks_[0].ev_g1;
    AK_CUDA(cudaStreamCreateWithFlags(&st2_, cudaStreamNonBlocking));
    AK_CUDA(cudaEventCreateWithFlags(&ev_fork_, cudaEventDisableTiming));
    AK_CUDA(cudaEventCreateWithFlags(&ev_join_, cudaEventDisableTiming));
    AK_CUDA(cudaStreamCreateWithFlags(&st_time_, cudaStreamNonBlocking));
    AK_CUDA(cudaEventCreateWithFlags(&ev_tfork_, cudaEventDisableTiming));
    AK_CUDA(cudaEventCreateWithFlags(&ev_tjoin_, cudaEventDisableTiming));
    AK_CUDA(cudaStreamSynchronize(ctx->stream));
    return AK_OK;
}

// mode: 0 store f32, 1 add into f32, 2 silu -> activation dtype
int Runner::gemm(const void* a, const void* wt, void* c, uint32_t m, uint32_t n, uint32_t k, int mode) {
    cudaStream_t st = ctx_->stream;
    if (w_->dtype == AK_F32) {
        uint32_t flags = mode == 1 ? GEMM_ADD : (mode == 2 ? GEMM_SILU : 0);
        return launch_gemm_f32(st, (const float*)a, (const float*)wt, (float*)c, m, n, k, flags);
    }
    uint32_t epi = mode == 1 ? AK_EPI_ADD_F32 : (mode == 2 ? AK_EPI_SILU_BF16 : AK_EPI_STORE_F32);
    return launch_gemm_bf16(st, a, wt, c, m, n, k, epi, n, true);
}

bool Runner::chunked_prefill_supported() const {
    const uint32_t hd = w_->cfg.dim / w_->cfg.num_heads;
    return w_->dtype == AK_BF16 && (hd == 64 || hd == 128) && tp_ == 1;
}

int Runner::launch_layers(uint32_t T, uint32_t n_pf_rows, uint32_t n_pf_seqs, uint32_t max_pf_len, bool any_decode,
                          uint32_t n_splits, bool capturing) {
    cudaStream_t st = ctx_->stream;
    const ak_model_config& c = w_->cfg;
    // With tensor parallelism (tp_ > 1) this rank holds heads_l_ heads (dq_ = heads_l_*hd columns of
    // q, k and v) and ffn_l_ ffn columns; the row-split out-proj / ffn-down products are partial
    // sums that go to tp_tmp_, are all-reduced, and are folded into the residual stream by the
    // rmsnorm that follows (h = hidden + sum, written back).
    const uint32_t D = c.dim, V = c.vocab_size, hd = D / c.num_heads, H = heads_l_, Dq = dq_, F = ffn_l_;
    const uint32_t dt = w_->dtype;
    const float scale = 1.0f / sqrtf((float)hd);
    const int32_t* rows = d_desc_ + d_.rows;
    const bool tp = tp_ > 1;
    bool pending = false;  // tp_tmp_ holds a reduced projection not yet added to hidden_
    int rc;
#define RC(x) do { rc = (x); if (rc) return rc; trace_mark(#x); } while (0)
    gtrace_capture_ = capturing && T == max_seqs_ && bank_ == 0;
    trace_mark("begin");
    if (!tp) {
        // One range of rows through every layer on one stream. Decode rows are [0, max_seqs_), prompt rows
        // follow; the two kinds never read each other's rows, so an admission step runs them as two
        // ranges on two streams, joined before the final norm.
        const size_t act = dt == AK_F32 ? 4 : 2;
        auto gemm_s = [&](cudaStream_t s, const void* a, const void* wt, void* cc, uint32_t m, uint32_t n, uint32_t k, int mode) -> int {
            if (dt == AK_F32) {
                const uint32_t flags = mode == 1 ? GEMM_ADD : (mode == 2 ? GEMM_SILU : 0);
                return launch_gemm_f32(s, (const float*)a, (const float*)wt, (float*)cc, m, n, k, flags);
            }
            const uint32_t epi = mode == 1 ? AK_EPI_ADD_F32 : (mode == 2 ? AK_EPI_SILU_BF16 : AK_EPI_STORE_F32);
            return launch_gemm_bf16(s, a, wt, cc, m, n, k, epi, n, true);
        };
        auto range = [&](cudaStream_t s, uint32_t r0, uint32_t nr, bool dec, bool pf) -> int {
            const int32_t* rw = rows + (size_t)r0 * 4;
            float* hid = hidden_ + (size_t)r0 * D;
            void* xn = (char*)xn_ + (size_t)r0 * D * act;
            float* qkv = qkv_ + (size_t)r0 * 3 * Dq;
            void* at = (char*)attn_ + (size_t)r0 * Dq * act;
            void* up = (char*)up_ + (size_t)r0 * F * act;
            RC(launch_embed_rows(s, rw + 0, 4, d_sampled_, w_->embedding, dt, hid, V, D, nr));
            for (uint32_t l = 0; l < c.num_layers; l++) {
                const auto& b = w_->blocks[l];
                RC(launch_rmsnorm(s, hid, b.norm_1, xn, dt, nullptr, nr, D, c.norm_eps));
                RC(gemm_s(s, xn, b.qkv, qkv, nr, 3 * Dq, D, 0));
                // Decode rows get their head split, RoPE and cache append inside the attention kernel (head sizes the
                // TMA kernel handles); the separate kernel then only serves the prompt rows of the range.
                const bool fuse = dec && attn_decode_fused_supported(hd);
                // decode rows and a prompt chunk in one range: the chunk's attention (a dozen CTAs walking the chunk's
                // keys one tile after the other) runs on the second stream BESIDE the decode attention, not after it
                const bool side_pf = dec && pf && n_pf_seqs && s == st && two_streams_;
                uint32_t a0 = r0, an = nr;
                if (fuse) { a0 = max_seqs_; an = (r0 + nr > max_seqs_) ? r0 + nr - max_seqs_ : 0; }
                if (an)
                    RC(launch_rope_kv_append(s, qkv_ + (size_t)a0 * 3 * Dq, rows + (size_t)a0 * 4 + 1, rows + (size_t)a0 * 4 + 2, 4,
                                             (char*)qbuf_ + (size_t)a0 * Dq * act, k_pool_[l], v_pool_[l], rope_table_, rope_len_, an, H, hd, 16, dt));
                if (side_pf) {
                    AK_CUDA(cudaEventRecord(ev_fork_, s));
                    AK_CUDA(cudaStreamWaitEvent(st2_, ev_fork_, 0));
                    RC(launch_attn_prefill_paged(st2_, qbuf_, k_pool_[l], v_pool_[l], d_desc_ + d_.block_tables, max_blocks_, d_desc_ + d_.pf_cu,
                                                 d_desc_ + d_.pf_slot, d_desc_ + d_.pf_pos0, attn_, n_pf_seqs, max_pf_len, max_seqs_, H, hd, 16, scale,
                                                 dt, max_rows_, n_blocks_));
                    AK_CUDA(cudaEventRecord(ev_join_, st2_));
                }
                if (dec) {  // rows [0, max_seqs_): this range starts at row 0
                    ak_attn_decode_params p{};
                    p.rows = max_seqs_; p.heads = H; p.head_dim = hd; p.block_size = 16; p.max_blocks_per_seq = max_blocks_;
                    p.scale = scale; p.kv_dtype = dt; p.n_splits = n_splits; p.pool_blocks = n_blocks_;
                    const bool timed = attn_timing_ && l == 0;
                    if (timed) RC(attn_time_mark(s, ev_attn0_, capturing));
                    // the kernels launched since the descriptor upload wrote nothing of the cache but, at most, each decode
                    // sequence's newest position (unfused) or a prompt's own blocks (the rows of another sequence)
                    g_attn_early = true;
                    if (fuse)
                        rc = launch_attn_decode_fused(s, qkv_, rope_table_, rope_len_, k_pool_[l], v_pool_[l], d_desc_ + d_.block_tables,
                                                      d_desc_ + d_.kv_lens, d_desc_ + d_.row_order, attn_, attn_scratch_, p, true);
                    else
                        rc = launch_attn_decode_paged(s, qbuf_, k_pool_[l], v_pool_[l], d_desc_ + d_.block_tables, d_desc_ + d_.kv_lens, attn_, attn_scratch_, p, true);
                    g_attn_early = false;
                    if (rc) return rc;
                    trace_mark("attn_decode");
                    if (timed) {
                        RC(attn_time_mark(s, ev_attn1_, capturing));
                        ev_valid_ = true;
                    }
                }
                if (side_pf) {
                    AK_CUDA(cudaStreamWaitEvent(s, ev_join_, 0));
                } else if (pf && n_pf_seqs) {  // prompt rows are addressed from row max_seqs_ of the full buffers
                    RC(launch_attn_prefill_paged(s, qbuf_, k_pool_[l], v_pool_[l], d_desc_ + d_.block_tables, max_blocks_, d_desc_ + d_.pf_cu,
                                                 d_desc_ + d_.pf_slot, d_desc_ + d_.pf_pos0, attn_, n_pf_seqs, max_pf_len, max_seqs_, H, hd, 16, scale,
                                                 dt, max_rows_, n_blocks_));
                }
                RC(gemm_s(s, at, b.out, hid, nr, D, Dq, 1));
                RC(launch_rmsnorm(s, hid, b.norm_2, xn, dt, nullptr, nr, D, c.norm_eps));
                RC(gemm_s(s, xn, b.up, up, nr, F, D, 2));
                RC(gemm_s(s, up, b.down, hid, nr, D, F, 1));
            }
            return AK_OK;
        };
        // A step of at most 128 rows (the decode rows plus one prompt chunk) is ONE row tile of every projection: the
        // prompt rows ride in the decode launches for free. Larger admission steps run the two kinds of rows as two
        // ranges on two streams.
        if (two_streams_ && any_decode && T > max_seqs_ && n_pf_seqs && T > 128) {
            AK_CUDA(cudaEventRecord(ev_fork_, st));
            AK_CUDA(cudaStreamWaitEvent(st2_, ev_fork_, 0));
            rc = range(st, 0, max_seqs_, true, false);
            if (rc) return rc;
            rc = range(st2_, max_seqs_, T - max_seqs_, false, true);
            if (rc) return rc;
            AK_CUDA(cudaEventRecord(ev_join_, st2_));
            AK_CUDA(cudaStreamWaitEvent(st, ev_join_, 0));
        } else {
            rc = range(st, 0, T, any_decode, true);
            if (rc) return rc;
        }
    } else {
        RC(launch_embed_rows(st, rows + 0, 4, d_sampled_, w_->embedding, dt, hidden_, V, D, T));
        for (uint32_t l = 0; l < c.num_layers; l++) {
            const auto& b = w_->blocks[l];
            if (pending) RC(launch_rmsnorm_rope_residual(st, hidden_, tp_tmp_, b.norm_1, xn_, nullptr, T, D, c.norm_eps, 0, dt));
            else RC(launch_rmsnorm(st, hidden_, b.norm_1, xn_, dt, nullptr, T, D, c.norm_eps));
            pending = false;
            RC(gemm(xn_, b.qkv, qkv_, T, 3 * Dq, D, 0));
            RC(launch_rope_kv_append(st, qkv_, rows + 1, rows + 2, 4, qbuf_, k_pool_[l], v_pool_[l], rope_table_, rope_len_, T, H, hd, 16, dt));
            if (any_decode) {
                ak_attn_decode_params p{};
                p.rows = max_seqs_; p.heads = H; p.head_dim = hd; p.block_size = 16; p.max_blocks_per_seq = max_blocks_;
                p.scale = scale; p.kv_dtype = dt; p.n_splits = n_splits; p.pool_blocks = n_blocks_;
                const bool timed = attn_timing_ && l == 0;
                if (timed) RC(attn_time_mark(st, ev_attn0_, capturing));
                g_attn_early = true;   // the append kernel just before wrote only the newest position of each decode sequence
                rc = launch_attn_decode_paged(st, qbuf_, k_pool_[l], v_pool_[l], d_desc_ + d_.block_tables, d_desc_ + d_.kv_lens, attn_, attn_scratch_, p, true);
                g_attn_early = false;
                if (rc) return rc;
                if (timed) {
                    RC(attn_time_mark(st, ev_attn1_, capturing));
                    ev_valid_ = true;
                }
            }
            if (n_pf_seqs) {
                RC(launch_attn_prefill_paged(st, qbuf_, k_pool_[l], v_pool_[l], d_desc_ + d_.block_tables, max_blocks_, d_desc_ + d_.pf_cu,
                                             d_desc_ + d_.pf_slot, d_desc_ + d_.pf_pos0, attn_, n_pf_seqs, max_pf_len, max_seqs_, H, hd, 16, scale, dt,
                                             max_rows_, n_blocks_));
            }
            if (tp) {
                RC(gemm(attn_, b.out, tp_tmp_, T, D, Dq, 0));
                RC(tp_all_reduce_f32(ctx_, tp_tmp_, (size_t)T * D));
                RC(launch_rmsnorm_rope_residual(st, hidden_, tp_tmp_, b.norm_2, xn_, nullptr, T, D, c.norm_eps, 0, dt));
            } else {
                RC(gemm(attn_, b.out, hidden_, T, D, Dq, 1));
                RC(launch_rmsnorm(st, hidden_, b.norm_2, xn_, dt, nullptr, T, D, c.norm_eps));
            }
            RC(gemm(xn_, b.up, up_, T, F, D, 2));
            if (tp) {
                RC(gemm(up_, b.down, tp_tmp_, T, D, F, 0));
                RC(tp_all_reduce_f32(ctx_, tp_tmp_, (size_t)T * D));
                pending = true;
            } else {
                RC(gemm(up_, b.down, hidden_, T, D, F, 1));
            }
        }
    }
    if (pending)  // fold the last ffn-down sum into the residual stream (the normalised output is not used)
        RC(launch_rmsnorm_rope_residual(st, hidden_, tp_tmp_, w_->final_norm, xn_, nullptr, T, D, c.norm_eps, 0, dt));
    RC(launch_rmsnorm(st, hidden_, w_->final_norm, xf_, dt, d_desc_ + d_.out_rows, max_seqs_, D, c.norm_eps));
    if (dt == AK_BF16) {
        // greedy argmax fused into the lm_head epilogue: logits are written only when someone reads them
        RC(launch_gemm_bf16_argmax(st, xf_, w_->lm_head, keep_logits_ ? logits_ : nullptr, logits_ld_, amax_val_, amax_idx_, max_seqs_, V, D));
        RC(launch_argmax_finish(st, amax_val_, amax_idx_, max_seqs_, amax_tiles_, d_desc_ + d_.out_rows, d_sampled_));
    } else {
        RC(gemm(xf_, w_->lm_head, logits_, max_seqs_, V, D, 0));
        RC(launch_argmax(st, logits_, max_seqs_, V, V, d_desc_ + d_.out_rows, d_sampled_));
    }
#undef RC
    (void)n_pf_rows;
    if (time_forked_) {  // the timing stream joins the step at its end
        time_forked_ = false;
        AK_CUDA(cudaEventRecord(ev_tjoin_, st_time_));
        AK_CUDA(cudaStreamWaitEvent(st, ev_tjoin_, 0));
    }
    return AK_OK;
}

// A timestamp at "everything launched on `s` so far has completed", taken on a side stream: the kernels on `s`
// keep their launch-to-launch overlap (an event recorded on `s` itself would sit between two kernels and cut
// the programmatic edge). Two marks around one launch measure from the completion of its predecessor, the
// moment its dependency wait returns, to its own completion.
int Runner::attn_time_mark(cudaStream_t s, cudaEvent_t ev, bool capturing) {
    AK_CUDA(cudaEventRecord(ev_tfork_, s));
    AK_CUDA(cudaStreamWaitEvent(st_time_, ev_tfork_, 0));
    if (capturing) AK_CUDA(cudaEventRecordWithFlags(ev, st_time_, cudaEventRecordExternal));
    else AK_CUDA(cudaEventRecord(ev, st_time_));
    time_forked_ = true;
    return AK_OK;
}

int Runner::run(uint32_t n_prefill_rows, uint32_t n_pf_seqs, uint32_t max_pf_len, bool any_decode, uint32_t max_kv_len) {
    AK_REQUIRE(n_prefill_rows <= max_pf_tokens_, AK_ERR_INVALID_ARG, "runner: %u prefill rows exceed the step budget %u", n_prefill_rows, max_pf_tokens_);
    AK_CUDA(cudaSetDevice(ctx_->device));
    cudaStream_t st = ctx_->stream;
    const uint32_t T = max_seqs_ + n_prefill_rows;
    const size_t bytes = ((size_t)d_.rows + (size_t)T * 4) * 4;
    attn_decode_row_order(h_kv_lens(), max_seqs_, heads_l_, w_->cfg.dim / w_->cfg.num_heads, w_->dtype, h_row_order());
    AK_CUDA(cudaMemcpyAsync(d_desc_, h_desc_, bytes, cudaMemcpyHostToDevice, st));
    // One split count per runner (from the longest sequence it can hold): eager and captured
    // steps then sum in the same order, so a sequence's tokens do not depend on its neighbours.
    (void)max_kv_len;
    const uint32_t n_splits = attn_decode_pick_splits(max_seqs_, heads_l_, w_->cfg.dim / w_->cfg.num_heads, w_->dtype, max_seq_len_);
    int rc = launch_layers(T, n_prefill_rows, n_pf_seqs, max_pf_len, any_decode, n_splits, false);
    if (rc) return rc;
    AK_CUDA(cudaMemcpyAsync(h_sampled_, d_sampled_, (size_t)max_seqs_ * 4, cudaMemcpyDeviceToHost, st));
    eager_steps++;
    h2d_bytes += bytes;
    d2h_bytes += (size_t)max_seqs_ * 4;
    return AK_OK;
}

static uint32_t pow2_bucket(uint32_t v, uint32_t lo) {
    uint32_t b = lo;
    while (b < v) b *= 2;
    return b;
}

// A step through a captured CUDA graph. Launch shapes are rounded up to a bucket
// (prefill rows: 0 or a power of two >= 64, capped at the step budget; prefilled sequences: a
// power of two), the padding rows / sequences are marked inactive in the descriptor, and one
// graph per bucket is captured on first use. Row results do not depend on the bucket (every
// kernel treats rows independently and the GEMM's K order is fixed per (n, k)).
int Runner::run_graph(uint32_t n_prefill_rows, uint32_t n_pf_seqs, uint32_t max_pf_len) {
    AK_REQUIRE(n_prefill_rows <= max_pf_tokens_ && n_pf_seqs <= max_seqs_, AK_ERR_INVALID_ARG, "runner: step exceeds its budget");
    AK_CUDA(cudaSetDevice(ctx_->device));
    cudaStream_t st = ctx_->stream;
    uint32_t rows_b = 0, seqs_b = 0, len_b = 0;
    if (n_prefill_rows) {
        rows_b = pow2_bucket(n_prefill_rows, 64);
        if (rows_b > max_pf_tokens_) rows_b = max_pf_tokens_;
        seqs_b = pow2_bucket(n_pf_seqs, 1);
        if (seqs_b > max_seqs_) seqs_b = max_seqs_;
        len_b = rows_b < max_seq_len_ ? rows_b : max_seq_len_;
        (void)max_pf_len;
        // mark the padding inactive
        RowInfo* rows = h_rows();
        for (uint32_t r = max_seqs_ + n_prefill_rows; r < max_seqs_ + rows_b; r++) rows[r] = {INT32_MIN, -1, -1, 0};
        int32_t* cu = h_pf_cu();
        int32_t* pfs = h_pf_slot();
        int32_t* p0 = h_pf_pos0();
        for (uint32_t i = n_pf_seqs; i < seqs_b; i++) { cu[i + 1] = cu[n_pf_seqs]; pfs[i] = 0; p0[i] = 0; }
    }
    attn_decode_row_order(h_kv_lens(), max_seqs_, heads_l_, w_->cfg.dim / w_->cfg.num_heads, w_->dtype, h_row_order());
    const uint64_t key = ((uint64_t)bank_ << 63) | ((uint64_t)rows_b << 32) | seqs_b;  // a graph bakes its bank's host buffers and events
    const uint32_t T = max_seqs_ + rows_b;
    const size_t bytes = ((size_t)d_.rows + (size_t)T * 4) * 4;
    const uint32_t n_splits = attn_decode_pick_splits(max_seqs_, heads_l_, w_->cfg.dim / w_->cfg.num_heads, w_->dtype, max_seq_len_);
    auto it = graphs_.find(key);
    if (it == graphs_.end()) {
        // one eager pass first (sets kernel attributes, surfaces faults outside capture); it IS this step
        AK_CUDA(cudaMemcpyAsync(d_desc_, h_desc_, bytes, cudaMemcpyHostToDevice, st));
        int rc = launch_layers(T, rows_b, seqs_b, len_b, true, n_splits, false);
        if (rc) return rc;
        AK_CUDA(cudaMemcpyAsync(h_sampled_, d_sampled_, (size_t)max_seqs_ * 4, cudaMemcpyDeviceToHost, st));
        AK_CUDA(cudaStreamSynchronize(st));
        eager_steps++;
        h2d_bytes += bytes;
        d2h_bytes += (size_t)max_seqs_ * 4;
        cudaGraph_t graph = nullptr;
        AK_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        cudaError_t e = cudaMemcpyAsync(d_desc_, h_desc_, bytes, cudaMemcpyHostToDevice, st);
        const unsigned long long l0 = g_launch_count;
        rc = (e == cudaSuccess) ? launch_layers(T, rows_b, seqs_b, len_b, true, n_splits, true) : AK_ERR_CUDA;
        StepGraph g;
        g.kernels = g_launch_count - l0;
        g.h2d = bytes;
        g_launch_count = l0;  // recorded into the graph, not launched
        if (rc == AK_OK) e = cudaMemcpyAsync(h_sampled_, d_sampled_, (size_t)max_seqs_ * 4, cudaMemcpyDeviceToHost, st);
        cudaError_t e2 = cudaStreamEndCapture(st, &graph);
        if (rc) return rc;
        if (e != cudaSuccess) return cuda_fail(e, "capture memcpy", __FILE__, __LINE__);
        if (e2 != cudaSuccess) return cuda_fail(e2, "cudaStreamEndCapture", __FILE__, __LINE__);
        AK_CUDA(cudaGraphInstantiate(&g.exec, graph, 0));
        cudaGraphDestroy(graph);
        graphs_[key] = g;
        if ((key << 1) == 0) graph_kernels = g.kernels;
        return AK_OK;
    }
    if (attn_timing_) AK_CUDA(cudaEventRecord(ev_g0_, st));
    const auto h0 = std::chrono::steady_clock::now();
    AK_CUDA(cudaGraphLaunch(it->second.exec, st));
    launch_host_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - h0).count();
    if (attn_timing_) { AK_CUDA(cudaEventRecord(ev_g1_, st)); ev_g_valid_ = true; }
    gtrace_ran_ = (key == 0);
    graph_launches++;
    g_launch_count += it->second.kernels;
    h2d_bytes += it->second.h2d;
    d2h_bytes += (size_t)max_seqs_ * 4;
    return AK_OK;
}

void Runner::set_bank(uint32_t b) {
    b &= 1u;
    if (b == bank_) return;
    banks_[bank_].ev_valid = ev_valid_;
    banks_[bank_].ev_g_valid = ev_g_valid_;
    bank_ = b;
    const Bank& k = banks_[b];
    h_desc_ = k.h_desc; h_sampled_ = k.h_sampled;
    ev_attn0_ = k.ev_attn0; ev_attn1_ = k.ev_attn1; ev_g0_ = k.ev_g0; ev_g1_ = k.ev_g1;
    ev_valid_ = k.ev_valid; ev_g_valid_ = k.ev_g_valid;
}

int Runner::mark_done() {
    AK_CUDA(cudaEventRecord(banks_[bank_].ev_done, ctx_->stream));
    return AK_OK;
}

int Runner::wait_bank(uint32_t b) {
    trace_dump();
    AK_CUDA(cudaEventSynchronize(banks_[b & 1u].ev_done));
    return AK_OK;
}

int Runner::run_decode_graph(uint32_t max_kv_len_hint) {
    (void)max_kv_len_hint;
    return run_graph(0, 0, 0);
}

void Runner::trace_mark(const char* label) {
    static int on = -1;
    if (on < 0) { const char* e = getenv("AK_TRACE"); on = (e && e[0] == '1') ? 1 : 0; }
    if (!on) return;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(ctx_->stream, &cs);
    if (cs == cudaStreamCaptureStatusActive) {
        if (!gtrace_capture_) return;
        cudaEvent_t ev;
        cudaEventCreate(&ev);
        gtrace_ev_.push_back(ev);
        gtrace_lbl_.push_back(label);
        cudaEventRecordWithFlags(ev, ctx_->stream, cudaEventRecordExternal);
        return;
    }
    if (trace_n_ == trace_ev_.size()) {
        cudaEvent_t ev;
        cudaEventCreate(&ev);
        trace_ev_.push_back(ev);
        trace_lbl_.push_back(label);
    }
    trace_lbl_[trace_n_] = label;
    cudaEventRecord(trace_ev_[trace_n_++], ctx_->stream);
}

void Runner::trace_dump() {
    if (gtrace_ran_ && gtrace_ev_.size() >= 2) {
        gtrace_ran_ = false;
        cudaStreamSynchronize(ctx_->stream);
        fprintf(stderr, "[ak gtrace] %zu launches\n", gtrace_ev_.size() - 1);
        for (size_t i = 1; i < gtrace_ev_.size(); i++) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, gtrace_ev_[i - 1], gtrace_ev_[i]) != cudaSuccess) { cudaGetLastError(); continue; }
            fprintf(stderr, "[ak gtrace] %8.2f us  %.60s\n", ms * 1e3f, gtrace_lbl_[i]);
        }
    }
    if (trace_n_ < 2) { trace_n_ = 0; return; }
    cudaStreamSynchronize(ctx_->stream);
    fprintf(stderr, "[ak trace] %zu launches\n", trace_n_ - 1);
    for (size_t i = 1; i < trace_n_; i++) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, trace_ev_[i - 1], trace_ev_[i]);
        fprintf(stderr, "[ak trace] %8.2f us  %.60s\n", ms * 1e3f, trace_lbl_[i]);
    }
    trace_n_ = 0;
}

int Runner::sync() {
    trace_dump();
    AK_CUDA(cudaStreamSynchronize(ctx_->stream));
    return AK_OK;
}

float Runner::last_step_gpu_ms() {
    if (!ev_g_valid_) return 0.0f;
    ev_g_valid_ = false;
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, ev_g0_, ev_g1_) != cudaSuccess) {
        cudaGetLastError();
        return 0.0f;
    }
    return ms;
}

float Runner::last_attn_ms() {
    if (!ev_valid_) return 0.0f;
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, ev_attn0_, ev_attn1_) != cudaSuccess) {
        cudaGetLastError();
        return 0.0f;
    }
    return ms;
}

int Runner::read_logits(uint32_t slot, float* host_out) {
    const uint32_t V = w_->cfg.vocab_size;
    AK_CUDA(cudaMemcpyAsync(host_out, logits_ + (size_t)slot * logits_ld_, (size_t)V * 4, cudaMemcpyDeviceToHost, ctx_->stream));
    AK_CUDA(cudaStreamSynchronize(ctx_->stream));
    return AK_OK;
}

int Runner::gather_cache(uint32_t layer, const int32_t* h_table, uint32_t len, float* k_out, float* v_out) {
    if (len == 0) return AK_OK;
    cudaStream_t st = ctx_->stream;
    const uint32_t D = w_->cfg.dim, H = w_->cfg.num_heads, hd = D / H;
    const uint32_t nb = (len + 15) / 16;
    int32_t* d_table = nullptr;
    float* d_out = nullptr;
    AK_CUDA(cudaMalloc((void**)&d_table, (size_t)nb * 4));
    AK_CUDA(cudaMalloc((void**)&d_out, (size_t)len * D * 4));
    AK_CUDA(cudaMemcpyAsync(d_table, h_table, (size_t)nb * 4, cudaMemcpyHostToDevice, st));
    int rc = AK_OK;
    for (int which = 0; which < 2 && rc == AK_OK; which++) {
        float* dst = which == 0 ? k_out : v_out;
        if (!dst) continue;
        rc = launch_gather_paged(st, which == 0 ? k_pool_[layer] : v_pool_[layer], w_->dtype, d_table, d_out, len, H, hd, 16);
        if (rc == AK_OK && cudaMemcpyAsync(dst, d_out, (size_t)len * D * 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) rc = AK_ERR_CUDA;
        if (rc == AK_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = AK_ERR_CUDA;
    }
    cudaFree(d_table);
    cudaFree(d_out);
    return rc;
}

}  // namespace ak
