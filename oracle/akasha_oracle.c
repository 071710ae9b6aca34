/*
 * akasha_oracle.c -- CPU restatement of the akasha-core Prefill/Decode inference math.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT. This file is the checker the CUDA library is compared
 * against. Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may load
 * it. Nothing in the shipped library links or calls it.
 *
 * Parity status: PINNED TO OUTPUTS OF THE REFERENCE'S OWN KERNEL CODE for every kernel whose source
 * the reference holds: make_ref.py (beside this file) compiles the CUDA C kernel strings of
 * src/shaders/cuda.rs unchanged (embedding, silu, rope, rope_offset, head_gather, attn_qk_cached,
 * softmax_rect, attn_av_cached, rmsnorm, cache_write, flash_attention) and writes their outputs
 * to tests/golden/reference_kernels.npz; tests/test_oracle_reference_kernels.py holds this file
 * to them, bit-exact except where the summation order differs (rmsnorm).
 * Still unpinned at the bit level: GEMM/GEMV (their arithmetic lives in the `wilupgu` crate,
 * absent from the reference tree; the order here is the one the reference's own test pins
 * within 1e-4, src/nn/ops/emit.rs:1449-1455) and the Rust host code (sampling), which are held
 * to the reference's in-test math and known answers (src/nn/ops/emit.rs:931-999, 1385-1411;
 * src/nn/sampling.rs:97-141).
 *
 * Each function cites the reference file:line whose arithmetic it follows. All arithmetic is
 * f32 with mul and add kept separate (compile with -ffp-contract=off): Rust never contracts
 * `a * b + c` into an fma. OpenMP is used only ACROSS independent output elements, so the
 * result of every element is the same whatever the thread count (threads=1 is the reference's
 * scalar loop order; threads=N is the timed CPU baseline).
 *
 * Optional bf16 emulation (`act_bf16`): activations are rounded to bfloat16 (round to nearest
 * even) at the points where the bf16 GPU engine stores them as bf16. The caller passes weights
 * that are already rounded.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define OR_EXPORT __attribute__((visibility("default")))

/* ---------------------------------------------------------------- helpers */

static inline float or_bf16_round(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN stays */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    u &= 0xffff0000u;
    float y;
    memcpy(&y, &u, 4);
    return y;
}

OR_EXPORT void or_round_bf16(float* x, uint64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; i++) x[i] = or_bf16_round(x[i]);
}

OR_EXPORT int or_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

OR_EXPORT void or_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Test-input generator shared by the reference's test modules (src/nn/ops/emit.rs:910-921):
 * 64-bit LCG, top 24 bits mapped to [-1, 1]. */
OR_EXPORT void or_lcg_fill(float* out, uint64_t n, uint64_t seed) {
    uint64_t state = seed + 0x9E3779B97F4A7C15ull;
    for (uint64_t i = 0; i < n; i++) {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        uint32_t bits = ((uint32_t)(state >> 40)) & 0x00FFFFFFu;
        out[i] = ((float)bits / (float)0x00FFFFFF) * 2.0f - 1.0f;
    }
}

/* ---------------------------------------------------------------- kernels */

/* src/shaders/cpu.rs:25-41 (and cuda.rs:21-29: an out-of-range id yields a zero row). */
OR_EXPORT void or_embedding(const uint32_t* tokens, const float* table, float* out,
                            uint32_t vocab, uint32_t dim, uint32_t seq_len) {
    for (uint32_t t = 0; t < seq_len; t++) {
        float* o = out + (size_t)t * dim;
        if (tokens[t] < vocab)
            memcpy(o, table + (size_t)tokens[t] * dim, (size_t)dim * 4);
        else
            memset(o, 0, (size_t)dim * 4);
    }
}

/* src/shaders/cpu.rs:205-222: ss summed in index order, x * rsqrt * w. */
OR_EXPORT void or_rmsnorm(const float* x, const float* w, float* out, uint32_t rows,
                          uint32_t size, float eps) {
#pragma omp parallel for schedule(static) if (rows > 1)
    for (int64_t r = 0; r < (int64_t)rows; r++) {
        const float* xr = x + (size_t)r * size;
        float* o = out + (size_t)r * size;
        float ss = 0.0f;
        for (uint32_t i = 0; i < size; i++) ss += xr[i] * xr[i];
        float rs = 1.0f / sqrtf((ss / (float)size) + eps);
        for (uint32_t i = 0; i < size; i++) o[i] = xr[i] * rs * w[i];
    }
}

/* C[m,n] (+)= A[m,k] @ B[k,n], all row-major (src/nn/ops/emit.rs:19,91). The arithmetic sits
 * in the absent wilupgu crate; the order fixed here is the one the reference test pins it
 * against (emit.rs:1449-1455): a single f32 accumulator from 0, k ascending, then `c0 + dot`
 * for the accumulate form. The j-inner loop below gives every (i,j) exactly that sequence. */
OR_EXPORT void or_matmul(const float* a, const float* b, float* c, uint32_t m, uint32_t n,
                         uint32_t k, int accumulate) {
    const uint32_t JB = 256;
    int64_t njb = (n + JB - 1) / JB;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < (int64_t)m; i++) {
        for (int64_t jb = 0; jb < njb; jb++) {
            uint32_t j0 = (uint32_t)jb * JB;
            uint32_t jn = (n - j0 < JB) ? (n - j0) : JB;
            float acc[256];
            for (uint32_t j = 0; j < jn; j++) acc[j] = 0.0f;
            const float* ar = a + (size_t)i * k;
            for (uint32_t kk = 0; kk < k; kk++) {
                float av = ar[kk];
                const float* br = b + (size_t)kk * n + j0;
                for (uint32_t j = 0; j < jn; j++) acc[j] += av * br[j];
            }
            float* cr = c + (size_t)i * n + j0;
            if (accumulate)
                for (uint32_t j = 0; j < jn; j++) cr[j] = cr[j] + acc[j];
            else
                for (uint32_t j = 0; j < jn; j++) cr[j] = acc[j];
        }
    }
}

/* src/shaders/cpu.rs:238-255 */
OR_EXPORT void or_head_gather(const float* src, float* dst, uint32_t seq_len, uint32_t full_dim,
                              uint32_t head_dim, uint32_t head_offset) {
    for (uint32_t r = 0; r < seq_len; r++)
        memcpy(dst + (size_t)r * head_dim, src + (size_t)r * full_dim + head_offset,
               (size_t)head_dim * 4);
}

/* src/shaders/cpu.rs:84-142 (rope: pos_offset = 0; rope_offset: pos_offset = pos).
 * Adjacent pairs, freq = 1/powf(10000, i/hd), angle = (float)abs_pos * freq. */
OR_EXPORT void or_rope(float* x, uint32_t seq_len, uint32_t dim, uint32_t head_dim,
                       uint32_t pos_offset) {
    uint32_t heads = dim / head_dim;
#pragma omp parallel for schedule(static) if (seq_len > 1)
    for (int64_t t = 0; t < (int64_t)seq_len; t++) {
        uint32_t abs_pos = (uint32_t)t + pos_offset;
        for (uint32_t d = 0; d < head_dim; d += 2) {
            float freq = 1.0f / powf(10000.0f, (float)d / (float)head_dim);
            float angle = (float)abs_pos * freq;
            float s = sinf(angle), c = cosf(angle);
            for (uint32_t h = 0; h < heads; h++) {
                size_t off = (size_t)t * dim + (size_t)h * head_dim + d;
                float x0 = x[off], x1 = x[off + 1];
                x[off] = x0 * c - x1 * s;
                x[off + 1] = x0 * s + x1 * c;
            }
        }
    }
}

/* src/shaders/cpu.rs:224-236 */
OR_EXPORT void or_cache_write(const float* src, float* cache, uint32_t row_count, uint32_t width,
                              uint32_t dst_row_offset) {
    memcpy(cache + (size_t)dst_row_offset * width, src, (size_t)row_count * width * 4);
}

/* src/shaders/cpu.rs:144-162: unscaled q.k, c ascending. */
OR_EXPORT void or_attn_qk_cached(const float* q, const float* k_cache, float* scores,
                                 uint32_t attn_len, uint32_t dim, uint32_t head_dim) {
    uint32_t heads = dim / head_dim;
#pragma omp parallel for schedule(static)
    for (int64_t h = 0; h < (int64_t)heads; h++) {
        const float* qh = q + (size_t)h * head_dim;
        for (uint32_t j = 0; j < attn_len; j++) {
            const float* kr = k_cache + (size_t)j * dim + (size_t)h * head_dim;
            float s = 0.0f;
            for (uint32_t c = 0; c < head_dim; c++) s += qh[c] * kr[c];
            scores[(size_t)h * attn_len + j] = s;
        }
    }
}

/* src/shaders/cpu.rs:180-203: max of scaled values, exp(x*scale - max), divide by the sum. */
OR_EXPORT void or_softmax_rect(float* x, uint32_t num_rows, uint32_t width, float scale) {
    for (uint32_t r = 0; r < num_rows; r++) {
        float* row = x + (size_t)r * width;
        float mx = -INFINITY;
        for (uint32_t i = 0; i < width; i++) {
            float v = row[i] * scale;
            mx = (v > mx) ? v : mx;
        }
        float sum = 0.0f;
        for (uint32_t i = 0; i < width; i++) {
            float e = expf(row[i] * scale - mx);
            row[i] = e;
            sum += e;
        }
        for (uint32_t i = 0; i < width; i++) row[i] /= sum;
    }
}

/* src/shaders/cpu.rs:164-178: out[d] = sum_j P[head(d), j] * V[j, d], j ascending. */
OR_EXPORT void or_attn_av_cached(const float* scores, const float* v_cache, float* out,
                                 uint32_t attn_len, uint32_t dim, uint32_t head_dim) {
    for (uint32_t d = 0; d < dim; d++) out[d] = 0.0f;
    uint32_t heads = dim / head_dim;
#pragma omp parallel for schedule(static)
    for (int64_t h = 0; h < (int64_t)heads; h++) {
        float* o = out + (size_t)h * head_dim;
        const float* p = scores + (size_t)h * attn_len;
        for (uint32_t j = 0; j < attn_len; j++) {
            const float* vr = v_cache + (size_t)j * dim + (size_t)h * head_dim;
            float pj = p[j];
            for (uint32_t c = 0; c < head_dim; c++) o[c] += pj * vr[c];
        }
    }
}

/* src/shaders/cpu.rs:63-69 */
OR_EXPORT void or_silu(float* x, uint64_t n) {
#pragma omp parallel for schedule(static) if (n > 65536)
    for (int64_t i = 0; i < (int64_t)n; i++) x[i] = x[i] / (1.0f + expf(-x[i]));
}

/* The reference CPU backend has no prefill-attention function (src/shaders/mod.rs:418-422,
 * `cpu: None`); the recurrence is the one of src/shaders/cuda.rs:633-685 and
 * src/shaders/fwd/flash_attention.wgsl:28-76: one (row, head) at a time, j ascending,
 * running max from -1e9, acc = acc*corr + p*v, final divide by the running sum. */
OR_EXPORT void or_flash_attention(const float* q, const float* k, const float* v, float* out,
                                  float* l_cache, uint32_t seq_len, uint32_t dim,
                                  uint32_t head_dim, float scale, uint32_t row_offset) {
    uint32_t heads = dim / head_dim;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int64_t row = 0; row < (int64_t)seq_len; row++) {
        for (int64_t h = 0; h < (int64_t)heads; h++) {
            float acc[128];
            size_t hoff = (size_t)h * head_dim;
            const float* qr = q + ((size_t)row_offset + row) * dim + hoff;
            for (uint32_t d = 0; d < head_dim; d++) acc[d] = 0.0f;
            float row_max = -1000000000.0f, row_sum = 0.0f;
            for (int64_t j = 0; j <= row; j++) {
                const float* kr = k + ((size_t)row_offset + j) * dim + hoff;
                const float* vr = v + ((size_t)row_offset + j) * dim + hoff;
                float s = 0.0f;
                for (uint32_t d = 0; d < head_dim; d++) s += qr[d] * kr[d];
                s *= scale;
                float new_max = fmaxf(row_max, s);
                float corr = expf(row_max - new_max);
                float p = expf(s - new_max);
                row_sum = row_sum * corr + p;
                for (uint32_t d = 0; d < head_dim; d++) acc[d] = acc[d] * corr + p * vr[d];
                row_max = new_max;
            }
            float* o = out + ((size_t)row_offset + row) * dim + hoff;
            for (uint32_t d = 0; d < head_dim; d++) o[d] = acc[d] / row_sum;
            if (l_cache) l_cache[(size_t)row * heads + h] = row_max + logf(row_sum);
        }
    }
}

/* src/nn/sampling.rs:83-91: the first index holding a strictly greater value wins. */
OR_EXPORT uint32_t or_argmax(const float* logits, uint32_t n) {
    uint32_t best = 0;
    for (uint32_t i = 0; i < n; i++)
        if (logits[i] > logits[best]) best = i;
    return best;
}

/* src/nn/sampling.rs:4-16 + 18-32 with temperature <= 0: repetition penalty then argmax. */
OR_EXPORT uint32_t or_sample_greedy(const float* logits, uint32_t n, const uint32_t* seen,
                                    uint32_t n_seen, float penalty) {
    float* l = (float*)malloc((size_t)n * 4);
    memcpy(l, logits, (size_t)n * 4);
    if (penalty != 1.0f) {
        uint8_t* mark = (uint8_t*)calloc(n, 1);
        for (uint32_t i = 0; i < n_seen; i++)
            if (seen[i] < n) mark[seen[i]] = 1;
        for (uint32_t i = 0; i < n; i++)
            if (mark[i]) l[i] = (l[i] > 0.0f) ? l[i] / penalty : l[i] * penalty;
        free(mark);
    }
    uint32_t r = or_argmax(l, n);
    free(l);
    return r;
}

/* src/nn/sampling.rs:18-81 with the uniform draw `r` supplied by the caller (the reference
 * calls an unseeded rand::random, sampling.rs:73). Candidates are ordered by logit descending;
 * equal logits by index ascending (the reference's sort_unstable_by leaves ties unspecified). */
typedef struct { float v; uint32_t i; } or_cand;
static int or_cand_cmp(const void* a, const void* b) {
    const or_cand* x = (const or_cand*)a; const or_cand* y = (const or_cand*)b;
    if (x->v > y->v) return -1;
    if (x->v < y->v) return 1;
    return (x->i > y->i) - (x->i < y->i);
}
OR_EXPORT uint32_t or_sample_token(const float* logits, uint32_t n, float temperature, uint32_t top_k, float top_p,
                                   const uint32_t* seen, uint32_t n_seen, float penalty, double r) {
    float* l = (float*)malloc((size_t)n * 4);
    memcpy(l, logits, (size_t)n * 4);
    if (penalty != 1.0f) {
        uint8_t* mark = (uint8_t*)calloc(n, 1);
        for (uint32_t i = 0; i < n_seen; i++)
            if (seen[i] < n) mark[seen[i]] = 1;
        for (uint32_t i = 0; i < n; i++)
            if (mark[i]) l[i] = (l[i] > 0.0f) ? l[i] / penalty : l[i] * penalty;
        free(mark);
    }
    if (temperature <= 0.0f) { uint32_t a = or_argmax(l, n); free(l); return a; }
    or_cand* c = (or_cand*)malloc(sizeof(or_cand) * n);
    for (uint32_t i = 0; i < n; i++) { c[i].v = l[i]; c[i].i = i; }
    qsort(c, n, sizeof(or_cand), or_cand_cmp);
    uint32_t m = n;
    if (top_k > 0 && top_k < n) m = top_k;
    double* p = (double*)malloc(sizeof(double) * m);
    double mx = (double)c[0].v, sum = 0.0;
    for (uint32_t j = 0; j < m; j++) { p[j] = exp(((double)c[j].v - mx) / (double)temperature); sum += p[j]; }
    for (uint32_t j = 0; j < m; j++) p[j] /= sum;
    if (top_p < 1.0f) {
        double cum = 0.0; uint32_t keep = m;
        for (uint32_t j = 0; j < m; j++) { cum += p[j]; if (cum >= (double)top_p) { keep = j + 1; break; } }
        m = keep;
        double s = 0.0;
        for (uint32_t j = 0; j < m; j++) s += p[j];
        for (uint32_t j = 0; j < m; j++) p[j] /= s;
    }
    uint32_t pick = c[m - 1].i;
    for (uint32_t j = 0; j < m; j++) { if (r < p[j]) { pick = c[j].i; break; } r -= p[j]; }
    free(p); free(c); free(l);
    return pick;
}

/* ---------------------------------------------------------------- model + session */

typedef struct {
    uint32_t vocab, dim, heads, layers, ffn;
    float eps;
    int act_bf16;
    /* Borrowed pointers, src/nn/weights.rs:158-171 `params()` order:
     * embedding, per block {norm_1, qkv_proj, out_proj, norm_2, ffn_up, ffn_down}, final_norm,
     * lm_head. Matrices are [in,out] row-major (src/nn/weights.rs:32-58). */
    const float** p;
} or_model;

typedef struct {
    or_model* m;
    uint32_t max_ctx, cur_len;
    float** k; /* per layer [max_ctx, dim], K stored after RoPE, V raw */
    float** v; /* (src/nn/inference_graphs.rs:511-543)                 */
} or_session;

/* status codes mirror AkashaError (src/lib.rs:10-17) */
enum { OR_OK = 0, OR_EMPTY_PROMPT = 1, OR_PROMPT_TOO_LONG = 2, OR_CONTEXT_FULL = 3, OR_NO_CACHE = 4,
       OR_CACHE_NOT_EMPTY = 5 };

OR_EXPORT or_model* or_model_create(uint32_t vocab, uint32_t dim, uint32_t heads, uint32_t layers,
                                    uint32_t ffn, float eps, const float* const* params,
                                    int act_bf16) {
    or_model* m = (or_model*)calloc(1, sizeof(or_model));
    m->vocab = vocab; m->dim = dim; m->heads = heads; m->layers = layers; m->ffn = ffn;
    m->eps = eps; m->act_bf16 = act_bf16;
    uint32_t np = 1 + 6 * layers + 2;
    m->p = (const float**)malloc(sizeof(float*) * np);
    for (uint32_t i = 0; i < np; i++) m->p[i] = params[i];
    return m;
}
OR_EXPORT void or_model_destroy(or_model* m) { if (m) { free(m->p); free(m); } }

OR_EXPORT or_session* or_session_create(or_model* m, uint32_t max_ctx) {
    or_session* s = (or_session*)calloc(1, sizeof(or_session));
    s->m = m; s->max_ctx = max_ctx; s->cur_len = 0;
    s->k = (float**)malloc(sizeof(float*) * m->layers);
    s->v = (float**)malloc(sizeof(float*) * m->layers);
    for (uint32_t l = 0; l < m->layers; l++) {
        s->k[l] = (float*)calloc((size_t)max_ctx * m->dim, 4);
        s->v[l] = (float*)calloc((size_t)max_ctx * m->dim, 4);
    }
    return s;
}
OR_EXPORT void or_session_destroy(or_session* s) {
    if (!s) return;
    for (uint32_t l = 0; l < s->m->layers; l++) { free(s->k[l]); free(s->v[l]); }
    free(s->k); free(s->v); free(s);
}
/* Cache::reset (src/nn/inference_graphs.rs:540-542): only the length goes back to 0. */
OR_EXPORT void or_session_reset(or_session* s) { s->cur_len = 0; }
OR_EXPORT uint32_t or_session_len(const or_session* s) { return s->cur_len; }
OR_EXPORT const float* or_session_k(const or_session* s, uint32_t layer) { return s->k[layer]; }
OR_EXPORT const float* or_session_v(const or_session* s, uint32_t layer) { return s->v[layer]; }

static void maybe_round(const or_model* m, float* x, uint64_t n) {
    if (m->act_bf16) or_round_bf16(x, n);
}

/* InferenceSession::prefill (src/nn/inference.rs:61-176) with build_prefill_layer
 * (src/nn/inference_graphs.rs:198-337). logits_out: [vocab]. all_hidden_out (optional):
 * hidden state after the last layer, [n, dim]. */
OR_EXPORT int or_prefill(or_session* s, const uint32_t* tokens, uint32_t n, float* logits_out) {
    or_model* m = s->m;
    if (n == 0) return OR_EMPTY_PROMPT;
    if (n > s->max_ctx) return OR_PROMPT_TOO_LONG;
    if (s->cur_len != 0) return OR_CACHE_NOT_EMPTY;
    uint32_t D = m->dim, F = m->ffn, hd = D / m->heads;
    float scale = 1.0f / sqrtf((float)hd);
    float* hidden = (float*)malloc((size_t)n * D * 4);
    float* norm = (float*)malloc((size_t)n * D * 4);
    float* qkv = (float*)malloc((size_t)n * 3 * D * 4);
    float* q = (float*)malloc((size_t)n * D * 4);
    float* k = (float*)malloc((size_t)n * D * 4);
    float* v = (float*)malloc((size_t)n * D * 4);
    float* att = (float*)malloc((size_t)n * D * 4);
    float* up = (float*)malloc((size_t)n * F * 4);
    or_embedding(tokens, m->p[0], hidden, m->vocab, D, n);
    for (uint32_t l = 0; l < m->layers; l++) {
        const float** bw = m->p + 1 + 6 * l;
        or_rmsnorm(hidden, bw[0], norm, n, D, m->eps);
        maybe_round(m, norm, (uint64_t)n * D);
        or_matmul(norm, bw[1], qkv, n, 3 * D, D, 0);
        or_head_gather(qkv, q, n, 3 * D, D, 0);
        or_head_gather(qkv, k, n, 3 * D, D, D);
        or_head_gather(qkv, v, n, 3 * D, D, 2 * D);
        or_rope(q, n, D, hd, 0);
        or_rope(k, n, D, hd, 0);
        maybe_round(m, q, (uint64_t)n * D);
        maybe_round(m, k, (uint64_t)n * D);
        maybe_round(m, v, (uint64_t)n * D);
        or_cache_write(k, s->k[l], n, D, 0);
        or_cache_write(v, s->v[l], n, D, 0);
        or_flash_attention(q, k, v, att, NULL, n, D, hd, scale, 0);
        maybe_round(m, att, (uint64_t)n * D);
        or_matmul(att, bw[2], hidden, n, D, D, 1);
        or_rmsnorm(hidden, bw[3], norm, n, D, m->eps);
        maybe_round(m, norm, (uint64_t)n * D);
        or_matmul(norm, bw[4], up, n, F, D, 0);
        or_silu(up, (uint64_t)n * F);
        maybe_round(m, up, (uint64_t)n * F);
        or_matmul(up, bw[5], hidden, n, D, F, 1);
    }
    /* last row only (src/nn/inference.rs:120-168) */
    float* last = hidden + (size_t)(n - 1) * D;
    or_rmsnorm(last, m->p[1 + 6 * m->layers], norm, 1, D, m->eps);
    maybe_round(m, norm, D);
    or_matmul(norm, m->p[2 + 6 * m->layers], logits_out, 1, m->vocab, D, 0);
    s->cur_len = n;
    free(hidden); free(norm); free(qkv); free(q); free(k); free(v); free(att); free(up);
    return OR_OK;
}

/* InferenceSession::decode_step (src/nn/inference.rs:178-262) with build_decode_layer
 * (src/nn/inference_graphs.rs:339-509): three-pass cached attention. */
OR_EXPORT int or_decode_step(or_session* s, uint32_t token, float* logits_out) {
    or_model* m = s->m;
    if (s->cur_len >= s->max_ctx) return OR_CONTEXT_FULL;
    uint32_t pos = s->cur_len, D = m->dim, F = m->ffn, hd = D / m->heads, L = pos + 1;
    float scale = 1.0f / sqrtf((float)hd);
    float* hidden = (float*)malloc((size_t)D * 4);
    float* norm = (float*)malloc((size_t)D * 4);
    float* qkv = (float*)malloc((size_t)3 * D * 4);
    float* q = (float*)malloc((size_t)D * 4);
    float* k = (float*)malloc((size_t)D * 4);
    float* v = (float*)malloc((size_t)D * 4);
    float* att = (float*)malloc((size_t)D * 4);
    float* up = (float*)malloc((size_t)F * 4);
    float* scores = (float*)malloc((size_t)m->heads * L * 4);
    or_embedding(&token, m->p[0], hidden, m->vocab, D, 1);
    for (uint32_t l = 0; l < m->layers; l++) {
        const float** bw = m->p + 1 + 6 * l;
        or_rmsnorm(hidden, bw[0], norm, 1, D, m->eps);
        maybe_round(m, norm, D);
        or_matmul(norm, bw[1], qkv, 1, 3 * D, D, 0);
        or_head_gather(qkv, q, 1, 3 * D, D, 0);
        or_head_gather(qkv, k, 1, 3 * D, D, D);
        or_head_gather(qkv, v, 1, 3 * D, D, 2 * D);
        or_rope(q, 1, D, hd, pos);
        or_rope(k, 1, D, hd, pos);
        maybe_round(m, q, D); maybe_round(m, k, D); maybe_round(m, v, D);
        or_cache_write(k, s->k[l], 1, D, pos);
        or_cache_write(v, s->v[l], 1, D, pos);
        or_attn_qk_cached(q, s->k[l], scores, L, D, hd);
        or_softmax_rect(scores, m->heads, L, scale);
        or_attn_av_cached(scores, s->v[l], att, L, D, hd);
        maybe_round(m, att, D);
        or_matmul(att, bw[2], hidden, 1, D, D, 1);
        or_rmsnorm(hidden, bw[3], norm, 1, D, m->eps);
        maybe_round(m, norm, D);
        or_matmul(norm, bw[4], up, 1, F, D, 0);
        or_silu(up, F);
        maybe_round(m, up, F);
        or_matmul(up, bw[5], hidden, 1, D, F, 1);
    }
    or_rmsnorm(hidden, m->p[1 + 6 * m->layers], norm, 1, D, m->eps);
    maybe_round(m, norm, D);
    or_matmul(norm, m->p[2 + 6 * m->layers], logits_out, 1, m->vocab, D, 0);
    s->cur_len = pos + 1;
    free(hidden); free(norm); free(qkv); free(q); free(k); free(v); free(att); free(up);
    free(scores);
    return OR_OK;
}

/* The harness rule for every model config: prefill, then `steps` greedy decode steps that do
 * NOT stop on eos (src/bin/diagnose.rs:799-804 drives the session the same way).
 * tokens_out[steps]; logits_out optional [steps+1, vocab] (row 0 = prefill logits).
 * Returns the number of tokens produced (less than `steps` only when the context fills). */
OR_EXPORT int or_generate_greedy(or_session* s, const uint32_t* prompt, uint32_t n, uint32_t steps,
                                 uint32_t* tokens_out, float* logits_out, int* status) {
    or_model* m = s->m;
    float* logits = (float*)malloc((size_t)m->vocab * 4);
    int rc = or_prefill(s, prompt, n, logits);
    if (status) *status = rc;
    if (rc != OR_OK) { free(logits); return 0; }
    if (logits_out) memcpy(logits_out, logits, (size_t)m->vocab * 4);
    uint32_t made = 0;
    for (uint32_t i = 0; i < steps; i++) {
        uint32_t next = or_argmax(logits, m->vocab);
        tokens_out[made++] = next;
        if (i + 1 == steps && !logits_out) break;
        rc = or_decode_step(s, next, logits);
        if (rc == OR_CONTEXT_FULL) break;
        if (logits_out) memcpy(logits_out + (size_t)(i + 1) * m->vocab, logits, (size_t)m->vocab * 4);
    }
    free(logits);
    return (int)made;
}

/* ---------------------------------------------------------------- paged-KV block allocator
 * The continuous-batching engine is new (the reference has no batching,
 * ARCHITECTURE.md:376-377); its slot rule is restated here so tests can check block tables:
 * free list starts ascending, the lowest free block is handed out first, a finished
 * sequence's blocks go back before the next admission.
 * slot(seq,pos) = table[pos / block] * block + pos % block. */
typedef struct { uint32_t n_blocks; uint8_t* used; } or_block_pool;

OR_EXPORT or_block_pool* or_pool_create(uint32_t n_blocks) {
    or_block_pool* p = (or_block_pool*)calloc(1, sizeof(or_block_pool));
    p->n_blocks = n_blocks;
    p->used = (uint8_t*)calloc(n_blocks, 1);
    return p;
}
OR_EXPORT void or_pool_destroy(or_block_pool* p) { if (p) { free(p->used); free(p); } }
OR_EXPORT int64_t or_pool_alloc(or_block_pool* p) {
    for (uint32_t i = 0; i < p->n_blocks; i++)
        if (!p->used[i]) { p->used[i] = 1; return i; }
    return -1;
}
OR_EXPORT void or_pool_free(or_block_pool* p, uint32_t b) { if (b < p->n_blocks) p->used[b] = 0; }
