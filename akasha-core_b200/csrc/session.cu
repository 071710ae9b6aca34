// Session level of the C ABI: the counterpart of `InferenceSession`
// (src/nn/inference.rs:13-327) on top of the ragged-batch runner with a single sequence slot.
// The KV cache is the runner's paged pool with the identity block table (block i = positions
// 16i .. 16i+15), so a gathered read reproduces the reference's contiguous [max_ctx, dim] rows.
#include <limits.h>

#include "model.h"

using namespace ak;

struct ak_session {
    ak_ctx* ctx = nullptr;
    ak_weights* w = nullptr;
    uint32_t max_ctx = 0;
    bool has_cache = false;  // `cache: Option<Cache>` (src/nn/inference.rs:18)
    uint32_t cur_len = 0;    // Cache::cur_len (src/nn/inference_graphs.rs:515)
    Runner runner;
    // sampled generation: the history (prompt + generated ids) on the device for the repetition penalty
    uint32_t* d_hist = nullptr;
    uint32_t* d_hist_off = nullptr;   // {0, history length}
    uint32_t hist_cap = 0;
    ~ak_session() {
        if (d_hist) cudaFree(d_hist);
        if (d_hist_off) cudaFree(d_hist_off);
    }
};

static void fill_identity_table(ak_session* s) {
    int32_t* t = s->runner.h_block_table(0);
    for (uint32_t i = 0; i < s->runner.max_blocks(); i++) t[i] = (int32_t)i;
}

extern "C" {

int ak_session_create(ak_ctx* ctx, ak_weights* w, uint32_t max_context_len, ak_session** out) {
    AK_REQUIRE(ctx && w && out, AK_ERR_INVALID_ARG, "ak_session_create: null pointer");
    AK_REQUIRE(max_context_len >= 1, AK_ERR_INVALID_ARG, "ak_session_create: max_context_len must be >= 1");
    ak_session* s = new ak_session();
    s->ctx = ctx;
    s->w = w;
    s->max_ctx = max_context_len;
    int rc = s->runner.init(ctx, w, 1, max_context_len, 0, max_context_len);
    if (rc) {
        delete s;
        return rc;
    }
    fill_identity_table(s);
    *out = s;
    return AK_OK;
}

int ak_session_destroy(ak_session* s) {
    delete s;
    return AK_OK;
}

int ak_session_attach_cache(ak_session* s) {
    AK_REQUIRE(s, AK_ERR_INVALID_ARG, "ak_session_attach_cache: null session");
    s->has_cache = true;
    s->cur_len = 0;
    return AK_OK;
}
int ak_session_take_cache(ak_session* s) {
    AK_REQUIRE(s, AK_ERR_INVALID_ARG, "ak_session_take_cache: null session");
    s->has_cache = false;
    s->cur_len = 0;
    return AK_OK;
}
int ak_session_reset_cache(ak_session* s) {
    AK_REQUIRE(s, AK_ERR_INVALID_ARG, "ak_session_reset_cache: null session");
    AK_REQUIRE(s->has_cache, AK_NO_CACHE, "no cache attached (call ak_session_attach_cache or generate first)");
    s->cur_len = 0;
    return AK_OK;
}
uint32_t ak_session_cur_len(const ak_session* s) { return s ? s->cur_len : 0; }

// src/nn/inference.rs:61-176
int ak_session_prefill(ak_session* s, const uint32_t* tokens, uint32_t n, float* logits_out, uint32_t* argmax_out) {
    AK_REQUIRE(s, AK_ERR_INVALID_ARG, "ak_session_prefill: null session");
    AK_REQUIRE(n != 0, AK_EMPTY_PROMPT, "prompt is empty");
    AK_REQUIRE(tokens, AK_ERR_INVALID_ARG, "ak_session_prefill: null tokens");
    AK_REQUIRE(n <= s->max_ctx, AK_PROMPT_TOO_LONG, "prompt is %u tokens, context window is %u", n, s->max_ctx);
    AK_REQUIRE(s->has_cache, AK_NO_CACHE, "no cache attached (call ak_session_attach_cache or generate first)");
    AK_REQUIRE(s->cur_len == 0, AK_CACHE_NOT_EMPTY,
               "prefill needs an empty cache, this one holds %u tokens (loop decode_step for a resumed cache)", s->cur_len);
    Runner& r = s->runner;
    RowInfo* rows = r.h_rows();
    rows[0] = {INT_MIN, -1, -1, 0};  // the slot's decode row is idle during a prefill
    for (uint32_t i = 0; i < n; i++) rows[1 + i] = {(int32_t)(tokens[i] & 0x7fffffffu), (int32_t)i, (int32_t)i, 0};
    for (uint32_t i = 0; i < n; i++)
        if (tokens[i] > 0x7fffffffu) rows[1 + i].tok_src = INT_MAX;  // out of any vocabulary: zero row
    r.h_kv_lens()[0] = 0;
    r.h_out_rows()[0] = (int32_t)n;  // row index of the last prompt token (only it feeds the lm_head)
    r.h_pf_cu()[0] = 0;
    r.h_pf_cu()[1] = (int32_t)n;
    r.h_pf_slot()[0] = 0;
    int rc = r.run(n, 1, n, false, n);
    if (rc) return rc;
    rc = r.sync();
    if (rc) return rc;
    s->cur_len = n;
    if (argmax_out) *argmax_out = r.h_sampled()[0];
    if (logits_out) return r.read_logits(0, logits_out);
    return AK_OK;
}

static int decode_one(ak_session* s, int32_t tok_src) {
    Runner& r = s->runner;
    const uint32_t pos = s->cur_len;
    r.h_rows()[0] = {tok_src, (int32_t)pos, (int32_t)pos, 0};
    r.h_kv_lens()[0] = (int32_t)(pos + 1);
    r.h_out_rows()[0] = 0;
    int rc = r.run_decode_graph(pos + 1);
    if (rc) return rc;
    s->cur_len = pos + 1;
    return AK_OK;
}

// src/nn/inference.rs:178-262
int ak_session_decode_step(ak_session* s, uint32_t token, float* logits_out, uint32_t* argmax_out) {
    AK_REQUIRE(s, AK_ERR_INVALID_ARG, "ak_session_decode_step: null session");
    AK_REQUIRE(s->has_cache, AK_NO_CACHE, "no cache attached (call ak_session_attach_cache or generate first)");
    AK_REQUIRE(s->cur_len < s->max_ctx, AK_CONTEXT_FULL, "context window is full (%u tokens)", s->max_ctx);
    int rc = decode_one(s, token > 0x7fffffffu ? INT_MAX : (int32_t)token);
    if (rc) return rc;
    rc = s->runner.sync();
    if (rc) return rc;
    if (argmax_out) *argmax_out = s->runner.h_sampled()[0];
    if (logits_out) return s->runner.read_logits(0, logits_out);
    return AK_OK;
}

// src/nn/inference.rs:264-326 with greedy sampling (src/nn/sampling.rs:30-32, 83-91).
int ak_session_generate_greedy(ak_session* s, const uint32_t* prompt, uint32_t n, uint32_t max_new, int stop_on_eos,
                               uint32_t* out_tokens, uint32_t* n_out) {
    AK_REQUIRE(s && n_out, AK_ERR_INVALID_ARG, "ak_session_generate_greedy: null pointer");
    *n_out = 0;
    AK_REQUIRE(n != 0, AK_EMPTY_PROMPT, "prompt is empty");
    AK_REQUIRE(prompt && (out_tokens || max_new == 0), AK_ERR_INVALID_ARG, "ak_session_generate_greedy: null pointer");
    if (!s->has_cache) {
        s->has_cache = true;
        s->cur_len = 0;
    }
    uint32_t next = 0;
    int rc;
    if (s->cur_len == 0) {
        rc = ak_session_prefill(s, prompt, n, nullptr, &next);
        if (rc) return rc;
    } else {
        for (uint32_t i = 0; i < n; i++) {
            rc = ak_session_decode_step(s, prompt[i], nullptr, &next);
            if (rc) return rc;
        }
    }
    const uint32_t eos = s->w->cfg.eos_token;
    for (uint32_t i = 0; i < max_new; i++) {
        out_tokens[(*n_out)++] = next;
        if (stop_on_eos && next == eos) break;
        if (s->cur_len >= s->max_ctx) break;  // out of context mid-generation: return what we have
        // the token just sampled stays on the device; only its id comes back
        rc = decode_one(s, -1);
        if (rc) return rc;
        rc = s->runner.sync();
        if (rc) return rc;
        next = s->runner.h_sampled()[0];
    }
    return AK_OK;
}

// src/nn/inference.rs:264-326 with sample_token (src/nn/sampling.rs:18-81) on the device.
int ak_session_generate(ak_session* s, const uint32_t* prompt, uint32_t n, uint32_t max_new, float temperature, uint32_t top_k,
                        float top_p, float repetition_penalty, uint64_t seed, int stop_on_eos, uint32_t* out_tokens, uint32_t* n_out) {
    AK_REQUIRE(s && n_out, AK_ERR_INVALID_ARG, "ak_session_generate: null pointer");
    *n_out = 0;
    AK_REQUIRE(n != 0, AK_EMPTY_PROMPT, "prompt is empty");
    AK_REQUIRE(prompt && (out_tokens || max_new == 0), AK_ERR_INVALID_ARG, "ak_session_generate: null pointer");
    cudaStream_t st = s->ctx->stream;
    AK_CUDA(cudaSetDevice(s->ctx->device));
    if (!s->has_cache) {
        s->has_cache = true;
        s->cur_len = 0;
    }
    // history = prompt, then every generated id (sample_token's `seen`, src/nn/inference.rs:303-317)
    const uint32_t need = n + max_new + 1;
    if (s->hist_cap < need) {
        if (s->d_hist) cudaFree(s->d_hist);
        s->d_hist = nullptr;
        s->hist_cap = 0;
        AK_CUDA(cudaMalloc((void**)&s->d_hist, (size_t)need * 4));
        s->hist_cap = need;
    }
    if (!s->d_hist_off) AK_CUDA(cudaMalloc((void**)&s->d_hist_off, 8));
    AK_CUDA(cudaMemcpyAsync(s->d_hist, prompt, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    uint32_t next = 0;
    int rc;
    if (s->cur_len == 0) {
        rc = ak_session_prefill(s, prompt, n, nullptr, &next);
        if (rc) return rc;
    } else {
        for (uint32_t i = 0; i < n; i++) {
            rc = ak_session_decode_step(s, prompt[i], nullptr, &next);
            if (rc) return rc;
        }
    }
    Runner& r = s->runner;
    const uint32_t V = s->w->cfg.vocab_size, eos = s->w->cfg.eos_token;
    uint32_t hist_len = n;
    for (uint32_t i = 0; i < max_new; i++) {
        // sample from the logits of the step just run; the id replaces the greedy one the step left for the next decode row
        const uint32_t off[2] = {0u, hist_len};
        AK_CUDA(cudaMemcpyAsync(s->d_hist_off, off, 8, cudaMemcpyHostToDevice, st));
        rc = launch_sample_rows(st, r.logits_dev(), 1, V, r.logits_ld(), s->d_hist, s->d_hist_off, repetition_penalty, temperature, top_k,
                                top_p, seed, i, nullptr, r.sampled_dev());
        if (rc) return rc;
        AK_CUDA(cudaMemcpyAsync(s->d_hist + hist_len, r.sampled_dev(), 4, cudaMemcpyDeviceToDevice, st));
        AK_CUDA(cudaMemcpyAsync(&next, r.sampled_dev(), 4, cudaMemcpyDeviceToHost, st));
        AK_CUDA(cudaStreamSynchronize(st));
        hist_len++;
        out_tokens[(*n_out)++] = next;
        if (stop_on_eos && next == eos) break;
        if (s->cur_len >= s->max_ctx) break;  // out of context mid-generation: return what we have
        rc = decode_one(s, -1);               // the sampled id is read on the device
        if (rc) return rc;
        rc = r.sync();
        if (rc) return rc;
    }
    return AK_OK;
}

int ak_session_read_cache(ak_session* s, uint32_t layer, float* k_out, float* v_out) {
    AK_REQUIRE(s, AK_ERR_INVALID_ARG, "ak_session_read_cache: null session");
    AK_REQUIRE(layer < s->w->cfg.num_layers, AK_ERR_INVALID_ARG, "ak_session_read_cache: layer %u out of range", layer);
    AK_REQUIRE(s->has_cache, AK_NO_CACHE, "no cache attached");
    return s->runner.gather_cache(layer, s->runner.h_block_table(0), s->cur_len, k_out, v_out);
}

}  // extern "C"
