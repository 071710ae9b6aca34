// HBM-bound row / element kernels of the Prefill/Decode path: the reference's single-emitter
// kernels (embedding, rmsnorm, head_gather, rope, rope_offset, cache_write, attn_qk_cached,
// softmax_rect, attn_av_cached, silu) and the fused forms the runtime uses
// (embed rows, rmsnorm(+residual)(+rope), split+rope+paged-append, greedy argmax).
#include "kernels.h"

namespace ak {

// ============================================================================ embedding
// src/shaders/cuda.rs:5-31: out[t,:] = table[tok[t],:]; an id >= vocab writes zeros.
__global__ void embedding_kernel(const uint32_t* __restrict__ tokens, const float* __restrict__ table,
                                 float* __restrict__ out, uint32_t vocab, uint32_t dim, uint32_t seq) {
    uint32_t t = blockIdx.x;
    if (t >= seq) return;
    uint32_t id = tokens[t];
    const float* src = table + (size_t)id * dim;
    float* dst = out + (size_t)t * dim;
    bool ok = id < vocab;
    if ((dim & 3u) == 0) {
        for (uint32_t i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            float4 v = ok ? *reinterpret_cast<const float4*>(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(dst + i) = v;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = ok ? src[i] : 0.0f;
    }
}

template <typename WT>
__global__ void embed_rows_kernel(const int32_t* __restrict__ tok_src, uint32_t idx_stride,
                                  const uint32_t* __restrict__ sampled, const WT* __restrict__ table,
                                  float* __restrict__ hidden, uint32_t vocab, uint32_t dim) {
    pdl_wait();
    pdl_trigger();
    uint32_t r = blockIdx.x;
    int32_t ts = tok_src[(size_t)r * idx_stride];
    // INT32_MIN marks an inactive row: it must not be decoded as a slot reference
    const bool active = ts != INT32_MIN;
    uint32_t id = 0;
    if (active) id = (ts >= 0) ? (uint32_t)ts : sampled[(uint32_t)(-(ts + 1))];
    bool ok = active && id < vocab;
    const WT* src = table + (size_t)(ok ? id : 0) * dim;
    float* dst = hidden + (size_t)r * dim;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = ok ? Cvt<WT>::to_f(src[i]) : 0.0f;
}

int launch_embed_rows(cudaStream_t st, const int32_t* tok_src, uint32_t idx_stride, const uint32_t* sampled,
                      const void* table, uint32_t table_dtype, float* hidden, uint32_t vocab, uint32_t dim,
                      uint32_t rows) {
    if (rows == 0) return AK_OK;
    if (table_dtype == AK_F32)
        AK_TRY(launch_k(embed_rows_kernel<float>, dim3(rows), dim3(256), 0, st, NO_CLUSTER, tok_src, idx_stride, sampled, (const float*)table, hidden, vocab, dim));
    else
        AK_TRY(launch_k(embed_rows_kernel<bf16>, dim3(rows), dim3(256), 0, st, NO_CLUSTER, tok_src, idx_stride, sampled, (const bf16*)table, hidden, vocab, dim));
    return AK_OK;
}

// ============================================================================ rmsnorm
// src/shaders/cuda.rs:421-456: y = x * (1/sqrt(ss/size + eps)) * w. One warp per row, the row is
// read once with 128-bit loads and held in registers when it fits (size <= 32*4*RCACHE).
template <typename OT, bool HAS_RES, bool ROPE, bool EARLY_W>
__global__ void rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ residual,
                                    const float* __restrict__ w, OT* __restrict__ y,
                                    const int32_t* __restrict__ row_map, const int32_t* __restrict__ positions,
                                    uint32_t rows, uint32_t size, float eps, uint32_t head_dim) {
    constexpr int RCACHE = 8;  // float4 per lane kept in registers -> size <= 1024 cached
    // EARLY_W (launches of a few rows inside a step's chain, where latency is everything): the norm weights do not
    // depend on the preceding kernel, so they are fetched (a trip to HBM: each layer's are read once per step) before
    // waiting for it. Launches of many rows keep the registers for occupancy instead.
    const bool vec = (size & 3u) == 0;
    float4 gcache[EARLY_W ? RCACHE : 1];
    if (EARLY_W && vec) {
#pragma unroll
        for (int c = 0; c < RCACHE; c++) {
            const uint32_t i = (threadIdx.x & 31) + 32u * c;
            gcache[EARLY_W ? c : 0] = i < (size >> 2) ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_wait();
    pdl_trigger();
    // RoPE frequencies 1 / 10000^(2i / head_dim): head_dim / 2 values for the whole launch, computed once per CTA
    __shared__ float s_freq[ROPE ? 128 : 1];
    const bool freq_tab = ROPE && head_dim <= 256;
    if (freq_tab) {
        for (uint32_t i = threadIdx.x; i < head_dim / 2; i += blockDim.x) s_freq[i] = 1.0f / powf(10000.0f, (float)(2 * i) / (float)head_dim);
        __syncthreads();
    }
    uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    uint32_t lane = threadIdx.x & 31;
    if (warp >= rows) return;
    int64_t src_row = row_map ? (int64_t)row_map[warp] : (int64_t)warp;
    OT* yr = y + (size_t)warp * size;
    if (src_row < 0) {
        for (uint32_t i = lane; i < size; i += 32) yr[i] = Cvt<OT>::from_f(0.0f);
        return;
    }
    float* xr = x + (size_t)src_row * size;
    const float* rr = HAS_RES ? residual + (size_t)src_row * size : nullptr;
    float4 cache[RCACHE];
    float ss = 0.0f;
    if (vec) {
        uint32_t nv = size >> 2;
#pragma unroll
        for (int c = 0; c < RCACHE; c++) {
            uint32_t i = lane + 32u * c;
            if (i < nv) {
                float4 v = reinterpret_cast<const float4*>(xr)[i];
                if (HAS_RES) {
                    float4 r = reinterpret_cast<const float4*>(rr)[i];
                    v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
                    reinterpret_cast<float4*>(xr)[i] = v;
                }
                cache[c] = v;
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        for (uint32_t i = lane + 32u * RCACHE; i < nv; i += 32) {
            float4 v = reinterpret_cast<const float4*>(xr)[i];
            if (HAS_RES) {
                float4 r = reinterpret_cast<const float4*>(rr)[i];
                v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
                reinterpret_cast<float4*>(xr)[i] = v;
            }
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (uint32_t i = lane; i < size; i += 32) {
            float v = xr[i];
            if (HAS_RES) { v += rr[i]; xr[i] = v; }
            ss += v * v;
        }
    }
    ss = warp_sum(ss);
    float rs = 1.0f / sqrtf((ss / (float)size) + eps);
    float pos = ROPE ? (float)positions[warp] : 0.0f;
    // RoPE factors of the two pairs (d0, d0+1), (d0+2, d0+3) of a float4. A lane visits float4 indices
    // lane, lane + 32, ...: 128 elements apart, so when head_dim divides 128 every one of them sits at the same
    // offset d0 inside its head and the transcendental work is done once per lane and row, not once per float4.
    const bool same_d0 = ROPE && (128u % head_dim) == 0;
    float hs0 = 0.f, hc0 = 1.f, hs1 = 0.f, hc1 = 1.f;
    auto factors = [&](uint32_t d0, float& s0, float& c0, float& s1, float& c1) {
        float f0 = freq_tab ? s_freq[d0 >> 1] : 1.0f / powf(10000.0f, (float)d0 / (float)head_dim);
        float f1 = freq_tab ? s_freq[(d0 >> 1) + 1] : 1.0f / powf(10000.0f, (float)(d0 + 2) / (float)head_dim);
        sincosf(pos * f0, &s0, &c0);
        sincosf(pos * f1, &s1, &c1);
    };
    if (same_d0 && head_dim <= 64) {
        // head_dim / 2 <= 32 distinct angles per row: each is evaluated by ONE lane (the same expressions as `factors`)
        // and handed to the lanes that need it, instead of every lane evaluating its own two
        const uint32_t half = head_dim >> 1, idx = lane & (half - 1);   // head_dim divides 128: a power of two
        const float f = freq_tab ? s_freq[idx] : 1.0f / powf(10000.0f, (float)(2 * idx) / (float)head_dim);
        float sn, cs;
        sincosf(pos * f, &sn, &cs);
        const uint32_t i0 = ((lane * 4) % head_dim) >> 1;
        hs0 = __shfl_sync(0xffffffffu, sn, i0); hc0 = __shfl_sync(0xffffffffu, cs, i0);
        hs1 = __shfl_sync(0xffffffffu, sn, i0 + 1); hc1 = __shfl_sync(0xffffffffu, cs, i0 + 1);
    } else if (same_d0) {
        factors((lane * 4) % head_dim, hs0, hc0, hs1, hc1);
    }

    auto emit4 = [&](uint32_t i4, float4 v, float4 g) {
        float o0 = v.x * rs * g.x, o1 = v.y * rs * g.y, o2 = v.z * rs * g.z, o3 = v.w * rs * g.w;
        if (ROPE) {
            float s0 = hs0, c0 = hc0, s1 = hs1, c1 = hc1;
            if (!same_d0) factors((i4 * 4) % head_dim, s0, c0, s1, c1);  // even d0, pairs (d0,d0+1) and (d0+2,d0+3)
            float a = o0 * c0 - o1 * s0, b = o0 * s0 + o1 * c0;
            float c = o2 * c1 - o3 * s1, d = o2 * s1 + o3 * c1;
            o0 = a; o1 = b; o2 = c; o3 = d;
        }
        if constexpr (sizeof(OT) == 4) {
            reinterpret_cast<float4*>(yr)[i4] = make_float4(o0, o1, o2, o3);
        } else {
            bf162 p0 = __floats2bfloat162_rn(o0, o1), p1 = __floats2bfloat162_rn(o2, o3);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&p0);
            pk.y = *reinterpret_cast<uint32_t*>(&p1);
            reinterpret_cast<uint2*>(yr)[i4] = pk;
        }
    };
    if (vec) {
        uint32_t nv = size >> 2;
#pragma unroll
        for (int c = 0; c < RCACHE; c++) {
            uint32_t i = lane + 32u * c;
            if (i < nv) emit4(i, cache[c], EARLY_W ? gcache[EARLY_W ? c : 0] : reinterpret_cast<const float4*>(w)[i]);
        }
        for (uint32_t i = lane + 32u * RCACHE; i < nv; i += 32) emit4(i, reinterpret_cast<const float4*>(xr)[i], reinterpret_cast<const float4*>(w)[i]);
    } else {
        // scalar tail path (ROPE needs even sizes and is only offered on the vector path)
        for (uint32_t i = lane; i < size; i += 32) yr[i] = Cvt<OT>::from_f(xr[i] * rs * w[i]);
    }
}

template <typename OT>
static int rmsnorm_dispatch(cudaStream_t st, float* x, const float* residual, const float* w, OT* y,
                            const int32_t* row_map, const int32_t* positions, uint32_t rows, uint32_t size,
                            float eps, uint32_t head_dim) {
    const int WARPS = 4;   // 8-warp CTAs (the RoPE frequency table shared by twice the rows) measured slower: 0.64 against 0.69 of peak
    dim3 grid(cdiv(rows, WARPS)), block(WARPS * 32);
    const bool rope = head_dim != 0, early = rows <= 1024;
#define AK_NORM_LAUNCH(RES, ROPE_, EARLY)                                                                                          \
    AK_TRY(launch_k(rmsnorm_rows_kernel<OT, RES, ROPE_, EARLY>, dim3(grid), dim3(block), 0, st, NO_CLUSTER, x, residual, w, y, row_map, \
                    positions, rows, size, eps, head_dim))
    if (residual && rope) { if (early) AK_NORM_LAUNCH(true, true, true); else AK_NORM_LAUNCH(true, true, false); }
    else if (residual) { if (early) AK_NORM_LAUNCH(true, false, true); else AK_NORM_LAUNCH(true, false, false); }
    else if (rope) { if (early) AK_NORM_LAUNCH(false, true, true); else AK_NORM_LAUNCH(false, true, false); }
    else { if (early) AK_NORM_LAUNCH(false, false, true); else AK_NORM_LAUNCH(false, false, false); }
#undef AK_NORM_LAUNCH
    return AK_OK;
}

int launch_rmsnorm(cudaStream_t st, const float* x, const float* w, void* y, uint32_t out_dtype,
                   const int32_t* row_map, uint32_t rows, uint32_t size, float eps) {
    if (rows == 0) return AK_OK;
    if (out_dtype == AK_F32)
        return rmsnorm_dispatch<float>(st, const_cast<float*>(x), nullptr, w, (float*)y, row_map, nullptr, rows, size, eps, 0);
    return rmsnorm_dispatch<bf16>(st, const_cast<float*>(x), nullptr, w, (bf16*)y, row_map, nullptr, rows, size, eps, 0);
}

int launch_rmsnorm_rope_residual(cudaStream_t st, float* x, const float* residual, const float* w, void* y,
                                 const int32_t* positions, uint32_t rows, uint32_t size, float eps,
                                 uint32_t head_dim, uint32_t out_dtype) {
    if (rows == 0) return AK_OK;
    if (head_dim != 0) {
        AK_REQUIRE((size & 3u) == 0 && (head_dim & 3u) == 0 && size % head_dim == 0 && positions, AK_ERR_INVALID_ARG,
                   "rmsnorm+rope: size and head_dim must be multiples of 4, size %% head_dim == 0, positions set");
    }
    if (out_dtype == AK_F32)
        return rmsnorm_dispatch<float>(st, x, residual, w, (float*)y, nullptr, positions, rows, size, eps, head_dim);
    return rmsnorm_dispatch<bf16>(st, x, residual, w, (bf16*)y, nullptr, positions, rows, size, eps, head_dim);
}

// ============================================================================ head_gather / cache_write
// src/shaders/cuda.rs:256-274
__global__ void head_gather_kernel(const float* __restrict__ src, float* __restrict__ dst, uint32_t seq,
                                   uint32_t full_dim, uint32_t head_dim, uint32_t head_offset) {
    uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t row = blockIdx.y;
    if (row >= seq || col >= head_dim) return;
    dst[(size_t)row * head_dim + col] = src[(size_t)row * full_dim + head_offset + col];
}
// src/shaders/cuda.rs:614-631 (the destination rows are contiguous: one flat copy)
__global__ void copy_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = src[i];
}

// ============================================================================ rope (emitter form)
// src/shaders/cuda.rs:98-123, 224-254. freq = 1/powf(10000, d/hd), angle = (float)pos * freq.
// The transcendental parts run in double and are rounded once, which lands on the host libm's
// f32 results (those are computed in double too) in all but rare double-rounding cases.
__global__ void rope_kernel(float* __restrict__ x, uint32_t seq, uint32_t dim, uint32_t head_dim, uint32_t pos_offset) {
    uint32_t half = head_dim >> 1;
    uint32_t pairs_per_row = dim >> 1;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)seq * pairs_per_row;
    if (idx >= total) return;
    uint32_t t = (uint32_t)(idx / pairs_per_row);
    uint32_t pr = (uint32_t)(idx % pairs_per_row);
    uint32_t d = (pr % half) * 2;
    float ratio = (float)d / (float)head_dim;
    float freq = 1.0f / (float)pow(10000.0, (double)ratio);
    float angle = (float)(t + pos_offset) * freq;
    float s = (float)sin((double)angle), c = (float)cos((double)angle);
    size_t off = (size_t)t * dim + (size_t)pr * 2;
    float x0 = x[off], x1 = x[off + 1];
    x[off] = x0 * c - x1 * s;
    x[off + 1] = x0 * s + x1 * c;
}

// ============================================================================ decode attention, emitter forms
// src/shaders/cuda.rs:349-369: one warp per (j, h), lanes over the head dimension.
__global__ void attn_qk_cached_kernel(const float* __restrict__ q, const float* __restrict__ kc,
                                      float* __restrict__ scores, uint32_t attn_len, uint32_t dim, uint32_t hd) {
    uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    uint32_t h = blockIdx.y;
    if (warp >= attn_len) return;
    const float* qh = q + (size_t)h * hd;
    const float* kr = kc + (size_t)warp * dim + (size_t)h * hd;
    float s = 0.0f;
    for (uint32_t c = lane; c < hd; c += 32) s += qh[c] * kr[c];
    s = warp_sum(s);
    if (lane == 0) scores[(size_t)h * attn_len + warp] = s;
}
// src/shaders/cuda.rs:391-419: one warp per row.
__global__ void softmax_rect_kernel(float* __restrict__ x, uint32_t rows, uint32_t width, float scale) {
    uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows) return;
    float* row = x + (size_t)warp * width;
    float mx = -INFINITY;
    for (uint32_t i = lane; i < width; i += 32) mx = fmaxf(mx, row[i] * scale);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (uint32_t i = lane; i < width; i += 32) {
        float e = expf(row[i] * scale - mx);
        row[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    for (uint32_t i = lane; i < width; i += 32) row[i] = row[i] / sum;
}
// src/shaders/cuda.rs:371-389: block = 32 d-columns x 8 j-slices, reduced through shared memory.
__global__ void attn_av_cached_kernel(const float* __restrict__ scores, const float* __restrict__ vc,
                                      float* __restrict__ out, uint32_t attn_len, uint32_t dim, uint32_t hd) {
    __shared__ float part[8][33];
    uint32_t d = blockIdx.x * 32 + threadIdx.x;
    float s = 0.0f;
    if (d < dim) {
        const float* p = scores + (size_t)(d / hd) * attn_len;
        for (uint32_t j = threadIdx.y; j < attn_len; j += 8) s += p[j] * vc[(size_t)j * dim + d];
    }
    part[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && d < dim) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) t += part[i][threadIdx.x];
        out[d] = t;
    }
}

// ============================================================================ silu
// src/shaders/cuda.rs:57-65, grid-stride so any length works (the reference needs a 2-D grid
// past 65535*256 elements, src/nn/ops/emit.rs:680-696).
__global__ void silu_kernel(float* __restrict__ x, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float v = x[i];
        x[i] = v / (1.0f + expf(-v));
    }
}
int launch_silu(cudaStream_t st, float* x, uint64_t n) {
    if (n == 0) return AK_OK;
    unsigned blocks = (unsigned)(cdiv64(n, 256) < B200_SMS * 16 ? cdiv64(n, 256) : B200_SMS * 16);
    silu_kernel<<<blocks, 256, 0, st>>>(x, n);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

// ============================================================================ split + RoPE + paged KV append
// One thread per 16-byte output chunk of one (token, head): VEC = 16/sizeof(T) elements.
template <typename T>
__global__ void rope_kv_append_kernel(const float* __restrict__ qkv, const int32_t* __restrict__ positions,
                                      const int32_t* __restrict__ slots, T* __restrict__ q_out,
                                      T* __restrict__ k_pool, T* __restrict__ v_pool,
                                      const float2* __restrict__ rope_table, uint32_t rope_table_len,
                                      uint32_t tokens, uint32_t heads, uint32_t hd, uint32_t bs, uint32_t idx_stride) {
    pdl_wait();
    pdl_trigger();
    constexpr int VEC = 16 / sizeof(T);
    uint32_t chunks_per_head = hd / VEC;
    uint32_t dim = heads * hd;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)tokens * heads * chunks_per_head;
    if (idx >= total) return;
    uint32_t c = (uint32_t)(idx % chunks_per_head);
    uint32_t h = (uint32_t)((idx / chunks_per_head) % heads);
    uint32_t t = (uint32_t)(idx / ((size_t)chunks_per_head * heads));
    int32_t slot = slots[(size_t)t * idx_stride];
    int32_t pos = positions[(size_t)t * idx_stride];
    if (pos < 0) return;  // inactive row
    uint32_t d0 = c * VEC;
    const float* row = qkv + (size_t)t * 3 * dim + (size_t)h * hd + d0;
    float qv[VEC], kv[VEC], vv[VEC];
#pragma unroll
    for (int i = 0; i < VEC; i += 4) {
        float4 a = *reinterpret_cast<const float4*>(row + i);
        float4 b = *reinterpret_cast<const float4*>(row + dim + i);
        float4 e = *reinterpret_cast<const float4*>(row + 2 * dim + i);
        qv[i] = a.x; qv[i + 1] = a.y; qv[i + 2] = a.z; qv[i + 3] = a.w;
        kv[i] = b.x; kv[i + 1] = b.y; kv[i + 2] = b.z; kv[i + 3] = b.w;
        vv[i] = e.x; vv[i + 1] = e.y; vv[i + 2] = e.z; vv[i + 3] = e.w;
    }
#pragma unroll
    for (int i = 0; i < VEC; i += 2) {
        uint32_t d = d0 + i;
        float cs, sn;
        if (rope_table && (uint32_t)pos < rope_table_len) {
            float2 f = rope_table[(size_t)pos * (hd >> 1) + (d >> 1)];
            cs = f.x; sn = f.y;
        } else {
            float freq = 1.0f / (float)pow(10000.0, (double)((float)d / (float)hd));
            float angle = (float)pos * freq;
            sn = (float)sin((double)angle);
            cs = (float)cos((double)angle);
        }
        rope_rotate(qv[i], qv[i + 1], cs, sn, qv[i], qv[i + 1]);
        rope_rotate(kv[i], kv[i + 1], cs, sn, kv[i], kv[i + 1]);
    }
    alignas(16) T qo[VEC], ko[VEC], vo[VEC];
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        qo[i] = Cvt<T>::from_f(qv[i]);
        ko[i] = Cvt<T>::from_f(kv[i]);
        vo[i] = Cvt<T>::from_f(vv[i]);
    }
    *reinterpret_cast<uint4*>(q_out + (size_t)t * dim + (size_t)h * hd + d0) = *reinterpret_cast<uint4*>(qo);
    if (slot >= 0) {
        uint32_t blk = (uint32_t)slot / bs, within = (uint32_t)slot % bs;
        size_t off = (((size_t)blk * heads + h) * bs + within) * hd + d0;
        *reinterpret_cast<uint4*>(k_pool + off) = *reinterpret_cast<uint4*>(ko);
        *reinterpret_cast<uint4*>(v_pool + off) = *reinterpret_cast<uint4*>(vo);
    }
}

int launch_rope_kv_append(cudaStream_t st, const float* qkv, const int32_t* positions, const int32_t* slots,
                          uint32_t idx_stride, void* q_out, void* k_pool, void* v_pool, const float2* rope_table,
                          uint32_t rope_table_len, uint32_t tokens, uint32_t heads, uint32_t head_dim,
                          uint32_t block_size, uint32_t kv_dtype) {
    if (tokens == 0) return AK_OK;
    // the kernels work on 16-byte chunks of the output: 4 f32 or 8 bf16 elements
    AK_REQUIRE(head_dim % (kv_dtype == AK_F32 ? 4 : 8) == 0, AK_ERR_UNSUPPORTED, "rope_kv_append: head_dim must be a multiple of %d for this dtype",
               kv_dtype == AK_F32 ? 4 : 8);
    if (kv_dtype == AK_F32) {
        size_t total = (size_t)tokens * heads * (head_dim / 4);
        AK_TRY(launch_k(rope_kv_append_kernel<float>, dim3((unsigned)cdiv64(total, 256)), dim3(256), 0, st, NO_CLUSTER, 
            qkv, positions, slots, (float*)q_out, (float*)k_pool, (float*)v_pool, rope_table, rope_table_len, tokens,
            heads, head_dim, block_size, idx_stride));
    } else {
        size_t total = (size_t)tokens * heads * (head_dim / 8);
        AK_TRY(launch_k(rope_kv_append_kernel<bf16>, dim3((unsigned)cdiv64(total, 256)), dim3(256), 0, st, NO_CLUSTER, 
            qkv, positions, slots, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, rope_table, rope_table_len, tokens,
            heads, head_dim, block_size, idx_stride));
    }
    return AK_OK;
}

// ============================================================================ greedy argmax
// src/nn/sampling.rs:83-91: the first index with a strictly greater value wins, i.e. among
// equal maxima the LOWEST index. One CTA per row, warp-shuffle reduction of (value, index).
__device__ __forceinline__ void argmax_combine(float& v, uint32_t& i, float ov, uint32_t oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}
__global__ void argmax_kernel(const float* __restrict__ logits, uint32_t n, uint32_t ld,
                              const int32_t* __restrict__ row_active, uint32_t* __restrict__ out_idx) {
    pdl_wait();
    pdl_trigger();
    uint32_t row = blockIdx.x;
    if (row_active && row_active[row] < 0) return;
    const float* l = logits + (size_t)row * ld;
    // NaN never compares greater, as in the reference loop; start from element 0.
    float best = l[0];
    uint32_t bi = 0;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = l[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_combine(best, bi, ov, oi);
    }
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = (lane < nw) ? sv[lane] : l[0];
        bi = (lane < nw) ? si[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_combine(best, bi, ov, oi);
        }
        if (lane == 0) out_idx[row] = bi;
    }
}
int launch_argmax(cudaStream_t st, const float* logits, uint32_t rows, uint32_t n, uint32_t ld,
                  const int32_t* row_active, uint32_t* out_idx) {
    if (rows == 0 || n == 0) return AK_OK;
    AK_TRY(launch_k(argmax_kernel, dim3(rows), dim3(1024), 0, st, NO_CLUSTER, logits, n, ld, row_active, out_idx));
    return AK_OK;
}

// Second stage of the argmax fused into the lm_head GEMM: one warp per row reduces the per-tile
// (max, first index) partials; equal maxima resolve to the lowest index.
__global__ void argmax_finish_kernel(const float* __restrict__ pv, const uint32_t* __restrict__ pi, uint32_t rows,
                                     uint32_t tiles, const int32_t* __restrict__ row_active, uint32_t* __restrict__ out_idx) {
    pdl_wait();
    pdl_trigger();
    uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    if (row_active && row_active[row] < 0) return;
    float best = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t t = lane; t < tiles; t += 32) {
        float v = pv[(size_t)row * tiles + t];
        uint32_t i = pi[(size_t)row * tiles + t];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_combine(best, bi, ov, oi);
    }
    if (lane == 0) out_idx[row] = (bi == 0xffffffffu) ? 0u : bi;
}
int launch_argmax_finish(cudaStream_t st, const float* part_val, const uint32_t* part_idx, uint32_t rows, uint32_t tiles,
                         const int32_t* row_active, uint32_t* out_idx) {
    if (rows == 0) return AK_OK;
    AK_TRY(launch_k(argmax_finish_kernel, dim3(cdiv(rows, 4)), dim3(128), 0, st, NO_CLUSTER, part_val, part_idx, rows, tiles, row_active, out_idx));
    return AK_OK;
}

// ============================================================================ conversions / layout
__global__ void f32_to_bf16_kernel(const float* __restrict__ s, bf16* __restrict__ d, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) d[i] = __float2bfloat16_rn(s[i]);
}
__global__ void bf16_to_f32_kernel(const bf16* __restrict__ s, float* __restrict__ d, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) d[i] = __bfloat162float(s[i]);
}
static unsigned stride_blocks(size_t n) {
    size_t b = cdiv64(n, 256);
    return (unsigned)(b < B200_SMS * 32 ? b : B200_SMS * 32);
}
int launch_f32_to_bf16(cudaStream_t st, const float* src, void* dst, uint64_t n) {
    if (!n) return AK_OK;
    f32_to_bf16_kernel<<<stride_blocks(n), 256, 0, st>>>(src, (bf16*)dst, n);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}
int launch_bf16_to_f32(cudaStream_t st, const void* src, float* dst, uint64_t n) {
    if (!n) return AK_OK;
    bf16_to_f32_kernel<<<stride_blocks(n), 256, 0, st>>>((const bf16*)src, dst, n);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}
// w_kn [k,n] f32  ->  wt_nk [n,k] bf16 through a 32x32 shared tile (both sides coalesced).
__global__ void transpose_to_bf16_kernel(const float* __restrict__ w, bf16* __restrict__ wt, uint32_t k, uint32_t n) {
    __shared__ float tile[32][33];
    uint32_t n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    for (uint32_t r = threadIdx.y; r < 32; r += blockDim.y) {
        uint32_t kk = k0 + r, nn = n0 + threadIdx.x;
        tile[r][threadIdx.x] = (kk < k && nn < n) ? w[(size_t)kk * n + nn] : 0.0f;
    }
    __syncthreads();
    for (uint32_t r = threadIdx.y; r < 32; r += blockDim.y) {
        uint32_t nn = n0 + r, kk = k0 + threadIdx.x;
        if (nn < n && kk < k) wt[(size_t)nn * k + kk] = __float2bfloat16_rn(tile[threadIdx.x][r]);
    }
}
__global__ void transpose_from_bf16_kernel(const bf16* __restrict__ wt, float* __restrict__ w, uint32_t k, uint32_t n) {
    __shared__ float tile[32][33];
    uint32_t n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    for (uint32_t r = threadIdx.y; r < 32; r += blockDim.y) {
        uint32_t nn = n0 + r, kk = k0 + threadIdx.x;
        tile[r][threadIdx.x] = (nn < n && kk < k) ? __bfloat162float(wt[(size_t)nn * k + kk]) : 0.0f;
    }
    __syncthreads();
    for (uint32_t r = threadIdx.y; r < 32; r += blockDim.y) {
        uint32_t kk = k0 + r, nn = n0 + threadIdx.x;
        if (kk < k && nn < n) w[(size_t)kk * n + nn] = tile[threadIdx.x][r];
    }
}
int launch_transpose_to_bf16(cudaStream_t st, const float* w_kn, void* wt_nk, uint32_t k, uint32_t n) {
    dim3 grid(cdiv(n, 32), cdiv(k, 32)), block(32, 8);
    transpose_to_bf16_kernel<<<grid, block, 0, st>>>(w_kn, (bf16*)wt_nk, k, n);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}
int launch_transpose_from_bf16(cudaStream_t st, const void* wt_nk, float* w_kn, uint32_t k, uint32_t n) {
    dim3 grid(cdiv(n, 32), cdiv(k, 32)), block(32, 8);
    transpose_from_bf16_kernel<<<grid, block, 0, st>>>((const bf16*)wt_nk, w_kn, k, n);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

// Counter-based normal generator (benchmark weights): splitmix64 of (seed, stream, element)
// -> two 24-bit uniforms -> Box-Muller.
__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ dst, size_t n, uint64_t seed, uint64_t stream_id, float mean, float std) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    uint64_t base = splitmix64(seed ^ splitmix64(stream_id * 0x632BE59BD9B4E019ull + 1));
    for (; i < n; i += stride) {
        uint64_t r = splitmix64(base + i);
        float u1 = ((float)((r >> 40) & 0xFFFFFF) + 1.0f) / 16777217.0f;
        float u2 = (float)((r >> 8) & 0xFFFFFF) / 16777216.0f;
        float z = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        dst[i] = Cvt<T>::from_f(mean + std * z);
    }
}
template <typename T>
__global__ void fill_normal_2d_kernel(T* __restrict__ dst, bool transposed, uint32_t lin, uint32_t lout, uint32_t gout,
                                      uint32_t row_off, uint32_t col_mode, uint32_t col_off, uint32_t blk_l, uint32_t blk_g,
                                      uint64_t seed, uint64_t stream_id, float mean, float std) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    const size_t n = (size_t)lin * lout;
    uint64_t base = splitmix64(seed ^ splitmix64(stream_id * 0x632BE59BD9B4E019ull + 1));
    for (; i < n; i += stride) {
        // i runs over the STORAGE order, so writes stay coalesced
        uint32_t r, c;
        if (transposed) { c = (uint32_t)(i / lin); r = (uint32_t)(i % lin); }
        else { r = (uint32_t)(i / lout); c = (uint32_t)(i % lout); }
        uint32_t gc = (col_mode == 3) ? (c / blk_l) * blk_g + col_off + c % blk_l : col_off + c;
        uint64_t g = (uint64_t)(r + row_off) * gout + gc;
        uint64_t rr = splitmix64(base + g);
        float u1 = ((float)((rr >> 40) & 0xFFFFFF) + 1.0f) / 16777217.0f;
        float u2 = (float)((rr >> 8) & 0xFFFFFF) / 16777216.0f;
        float z = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        dst[i] = Cvt<T>::from_f(mean + std * z);
    }
}
int launch_fill_normal_2d(cudaStream_t st, void* dst, uint32_t dtype, bool transposed, uint32_t lin, uint32_t lout,
                          uint32_t gout, uint32_t row_off, uint32_t col_mode, uint32_t col_off, uint32_t blk_l,
                          uint32_t blk_g, uint64_t seed, uint64_t stream_id, float mean, float std) {
    size_t n = (size_t)lin * lout;
    if (!n) return AK_OK;
    if (dtype == AK_F32)
        fill_normal_2d_kernel<float><<<stride_blocks(n), 256, 0, st>>>((float*)dst, transposed, lin, lout, gout, row_off, col_mode, col_off, blk_l, blk_g, seed, stream_id, mean, std);
    else
        fill_normal_2d_kernel<bf16><<<stride_blocks(n), 256, 0, st>>>((bf16*)dst, transposed, lin, lout, gout, row_off, col_mode, col_off, blk_l, blk_g, seed, stream_id, mean, std);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

int launch_fill_normal(cudaStream_t st, void* dst, uint32_t dtype, uint64_t n, uint64_t seed, uint64_t stream_id,
                       float mean, float std) {
    if (!n) return AK_OK;
    if (dtype == AK_F32)
        fill_normal_kernel<float><<<stride_blocks(n), 256, 0, st>>>((float*)dst, n, seed, stream_id, mean, std);
    else
        fill_normal_kernel<bf16><<<stride_blocks(n), 256, 0, st>>>((bf16*)dst, n, seed, stream_id, mean, std);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

template <typename T>
__global__ void gather_paged_kernel(const T* __restrict__ pool, const int32_t* __restrict__ table,
                                    float* __restrict__ out, uint32_t len, uint32_t heads, uint32_t hd, uint32_t bs) {
    uint32_t dim = heads * hd;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)len * dim) return;
    uint32_t pos = (uint32_t)(idx / dim), col = (uint32_t)(idx % dim);
    uint32_t h = col / hd, d = col % hd;
    uint32_t blk = (uint32_t)table[pos / bs], within = pos % bs;
    out[idx] = Cvt<T>::to_f(pool[(((size_t)blk * heads + h) * bs + within) * hd + d]);
}
int launch_gather_paged(cudaStream_t st, const void* pool, uint32_t kv_dtype, const int32_t* block_table,
                        float* out, uint32_t len, uint32_t heads, uint32_t head_dim, uint32_t block_size) {
    if (!len) return AK_OK;
    size_t total = (size_t)len * heads * head_dim;
    if (kv_dtype == AK_F32)
        gather_paged_kernel<float><<<(unsigned)cdiv64(total, 256), 256, 0, st>>>((const float*)pool, block_table, out, len, heads, head_dim, block_size);
    else
        gather_paged_kernel<bf16><<<(unsigned)cdiv64(total, 256), 256, 0, st>>>((const bf16*)pool, block_table, out, len, heads, head_dim, block_size);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

}  // namespace ak

// ============================================================================ C ABI, emitter level
using namespace ak;

extern "C" {

int ak_embedding(void* stream, const uint32_t* tokens, const float* table, float* out, ak_embedding_meta m) {
    AK_REQUIRE(tokens && table && out, AK_ERR_INVALID_ARG, "ak_embedding: null pointer");
    if (m.seq_len == 0) return AK_OK;
    embedding_kernel<<<m.seq_len, 256, 0, as_stream(stream)>>>(tokens, table, out, m.vocab_size, m.dim, m.seq_len);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

int ak_rmsnorm(void* stream, const float* x, const float* w, float* y, ak_norm_meta m) {
    AK_REQUIRE(x && w && y, AK_ERR_INVALID_ARG, "ak_rmsnorm: null pointer");
    return launch_rmsnorm(as_stream(stream), x, w, y, AK_F32, nullptr, m.seq_len, m.size, m.eps);
}

int ak_head_gather(void* stream, const float* src, float* dst, ak_head_move_meta m) {
    AK_REQUIRE(src && dst, AK_ERR_INVALID_ARG, "ak_head_gather: null pointer");
    if (m.seq_len == 0 || m.head_dim == 0) return AK_OK;
    dim3 grid(cdiv(m.head_dim, 256), m.seq_len);
    head_gather_kernel<<<grid, 256, 0, as_stream(stream)>>>(src, dst, m.seq_len, m.full_dim, m.head_dim, m.head_offset);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

static int rope_common(void* stream, float* x, uint32_t seq, uint32_t dim, uint32_t hd, uint32_t pos) {
    AK_REQUIRE(x, AK_ERR_INVALID_ARG, "ak_rope: null pointer");
    AK_REQUIRE(hd >= 2 && (hd & 1u) == 0 && dim % hd == 0, AK_ERR_INVALID_ARG, "ak_rope: head_dim must be even and divide dim");
    size_t total = (size_t)seq * (dim / 2);
    if (!total) return AK_OK;
    rope_kernel<<<(unsigned)cdiv64(total, 256), 256, 0, as_stream(stream)>>>(x, seq, dim, hd, pos);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}
int ak_rope(void* stream, float* x, ak_rope_meta m) { return rope_common(stream, x, m.seq_len, m.dim, m.head_dim, 0); }
int ak_rope_offset(void* stream, float* x, ak_rope_offset_meta m) {
    return rope_common(stream, x, m.seq_len, m.dim, m.head_dim, m.pos);
}

int ak_cache_write(void* stream, const float* src, float* cache, ak_cache_write_meta m) {
    AK_REQUIRE(src && cache, AK_ERR_INVALID_ARG, "ak_cache_write: null pointer");
    size_t n = (size_t)m.row_count * m.width;
    if (!n) return AK_OK;
    copy_f32_kernel<<<stride_blocks(n), 256, 0, as_stream(stream)>>>(src, cache + (size_t)m.dst_row_offset * m.width, n);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

int ak_attn_qk_cached(void* stream, const float* q, const float* k_cache, float* scores, ak_attn_cached_meta m) {
    AK_REQUIRE(q && k_cache && scores, AK_ERR_INVALID_ARG, "ak_attn_qk_cached: null pointer");
    AK_REQUIRE(m.head_dim && m.dim % m.head_dim == 0, AK_ERR_INVALID_ARG, "ak_attn_qk_cached: bad head_dim");
    if (!m.attn_len) return AK_OK;
    dim3 grid(cdiv(m.attn_len, 8), m.dim / m.head_dim);
    attn_qk_cached_kernel<<<grid, 256, 0, as_stream(stream)>>>(q, k_cache, scores, m.attn_len, m.dim, m.head_dim);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

int ak_softmax_rect(void* stream, float* x, ak_softmax_rect_meta m) {
    AK_REQUIRE(x, AK_ERR_INVALID_ARG, "ak_softmax_rect: null pointer");
    if (!m.num_rows || !m.width) return AK_OK;
    softmax_rect_kernel<<<cdiv(m.num_rows, 4), 128, 0, as_stream(stream)>>>(x, m.num_rows, m.width, m.scale);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

int ak_attn_av_cached(void* stream, const float* scores, const float* v_cache, float* out, ak_attn_cached_meta m) {
    AK_REQUIRE(scores && v_cache && out, AK_ERR_INVALID_ARG, "ak_attn_av_cached: null pointer");
    AK_REQUIRE(m.head_dim && m.dim % m.head_dim == 0, AK_ERR_INVALID_ARG, "ak_attn_av_cached: bad head_dim");
    dim3 grid(cdiv(m.dim, 32)), block(32, 8);
    attn_av_cached_kernel<<<grid, block, 0, as_stream(stream)>>>(scores, v_cache, out, m.attn_len, m.dim, m.head_dim);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

int ak_silu(void* stream, float* x, uint32_t n) {
    AK_REQUIRE(x || n == 0, AK_ERR_INVALID_ARG, "ak_silu: null pointer");
    return launch_silu(as_stream(stream), x, n);
}

int ak_argmax(void* stream, const float* logits, uint32_t rows, uint32_t n, uint32_t* out_idx) {
    AK_REQUIRE(logits && out_idx, AK_ERR_INVALID_ARG, "ak_argmax: null pointer");
    return launch_argmax(as_stream(stream), logits, rows, n, n, nullptr, out_idx);
}

int ak_rope_kv_append(void* stream, const float* qkv, const int32_t* positions, const int32_t* slots, void* q_out,
                      void* k_pool, void* v_pool, uint32_t tokens, uint32_t heads, uint32_t head_dim,
                      uint32_t block_size, uint32_t kv_dtype) {
    AK_REQUIRE(qkv && positions && slots && q_out && k_pool && v_pool, AK_ERR_INVALID_ARG, "ak_rope_kv_append: null pointer");
    AK_REQUIRE(kv_dtype <= AK_BF16, AK_ERR_INVALID_ARG, "ak_rope_kv_append: bad dtype");
    return launch_rope_kv_append(as_stream(stream), qkv, positions, slots, 1, q_out, k_pool, v_pool, nullptr, 0, tokens,
                                 heads, head_dim, block_size, kv_dtype);
}

int ak_rmsnorm_rope_residual(void* stream, float* x, const float* residual, const float* w, void* y,
                             const int32_t* positions, uint32_t rows, uint32_t size, float eps, uint32_t head_dim,
                             uint32_t out_dtype) {
    AK_REQUIRE(x && w && y, AK_ERR_INVALID_ARG, "ak_rmsnorm_rope_residual: null pointer");
    AK_REQUIRE(out_dtype <= AK_BF16, AK_ERR_INVALID_ARG, "ak_rmsnorm_rope_residual: bad dtype");
    return launch_rmsnorm_rope_residual(as_stream(stream), x, residual, w, y, positions, rows, size, eps, head_dim, out_dtype);
}

int ak_transpose_to_bf16(void* stream, const float* w_kn, void* wt_nk, uint32_t k, uint32_t n) {
    AK_REQUIRE(w_kn && wt_nk, AK_ERR_INVALID_ARG, "ak_transpose_to_bf16: null pointer");
    return launch_transpose_to_bf16(as_stream(stream), w_kn, wt_nk, k, n);
}
int ak_f32_to_bf16(void* stream, const float* src, void* dst, uint64_t n) {
    return launch_f32_to_bf16(as_stream(stream), src, dst, n);
}
int ak_bf16_to_f32(void* stream, const void* src, float* dst, uint64_t n) {
    return launch_bf16_to_f32(as_stream(stream), src, dst, n);
}

}  // extern "C"

// ============================================================================ on-device sampler
// `sample_token` (src/nn/sampling.rs:18-81) on the device, one CTA per sequence: repetition
// penalty over the distinct seen ids (divide positive logits, multiply the others), then
// temperature / top-k / top-p sampling with the probabilities formed in f64 as the reference does.
// The reference draws its uniform number from an unseeded generator (sampling.rs:73); here it comes
// from a counter-based generator over (seed, step, row), so a run can be reproduced. Candidates
// are ordered by (logit descending, index ascending); the reference's unstable sort leaves the
// order of EQUAL logits unspecified. temperature <= 0 is the greedy argmax of the penalised logits.
namespace ak {

constexpr int SMP_THREADS = 1024;
constexpr int SMP_MAX_K = 1024;

__device__ __forceinline__ uint64_t smp_mix(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// ---- no top-k truncation (top_k == 0, src/nn/sampling.rs:41-43): the candidate list is the whole vocabulary.
// Instead of sorting 50k (logit, id) pairs, the two places where the reference walks its sorted list -- the top-p
// cut and the draw -- are found by bisection on the logit value: "the mass of every candidate whose logit is
// >= x" is a block-wide sum, and 32 such sums locate, bit by bit, the value at which the walk would stop; ties at
// that value are then taken in index order, as the sorted list orders them.
// Order-preserving map float -> uint32 (larger float, larger key); NaN sorts below everything.
__device__ __forceinline__ uint32_t smp_key(float v) {
    if (v != v) return 0u;
    const uint32_t b = __float_as_uint(v);
    const uint32_t k = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return k == 0u ? 1u : k;
}
// Sum over the row of exp((v - mx) / T) for candidates with key >= theta (all threads get the result), and their count.
__device__ double smp_mass_ge(const float* srow, uint32_t n, uint32_t theta, double mx, double T, double* red, uint32_t* cnt_out) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    double acc = 0.0;
    uint32_t cnt = 0;
    for (uint32_t i = tid; i < n; i += SMP_THREADS) {
        const float v = srow[i];
        if (smp_key(v) >= theta && v == v) { acc += exp(((double)v - mx) / T); cnt++; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { acc += __shfl_xor_sync(0xffffffffu, acc, o); cnt += __shfl_xor_sync(0xffffffffu, cnt, o); }
    __syncthreads();   // red is reused between calls
    if (lane == 0) { red[warp] = acc; red[32 + warp] = (double)cnt; }
    __syncthreads();
    double tot = 0.0, c = 0.0;
    for (int w = 0; w < SMP_THREADS / 32; w++) { tot += red[w]; c += red[32 + w]; }   // same order in every thread
    if (cnt_out) *cnt_out = (uint32_t)c;
    return tot;
}
// Largest key theta with mass(theta) >= target (strict == false) or > target (strict == true); mass(0) covers the row.
__device__ uint32_t smp_bisect(const float* srow, uint32_t n, double target, bool strict, double mx, double T, double* red) {
    uint32_t theta = 0;
    for (int b = 31; b >= 0; b--) {
        const uint32_t t2 = theta | (1u << b);
        const double m = smp_mass_ge(srow, n, t2, mx, T, red, nullptr);
        if (strict ? (m > target) : (m >= target)) theta = t2;
    }
    return theta;
}
// The whole-vocabulary sampler; called by every thread of the CTA, returns the pick in every thread.
__device__ uint32_t smp_sample_untruncated(const float* srow, uint32_t n, float temperature, float top_p, double r, double* red,
                                           uint32_t* scan) {
    const uint32_t tid = threadIdx.x;
    const double T = (double)temperature;
    // max of the row = the first candidate
    float best = -INFINITY;
    for (uint32_t i = tid; i < n; i += SMP_THREADS) best = fmaxf(best, srow[i]);
    best = warp_max(best);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = (double)best;
    __syncthreads();
    double mx = red[0];
    for (int w = 1; w < SMP_THREADS / 32; w++) mx = fmax(mx, red[w]);
    uint32_t n_all = 0;
    const double total = smp_mass_ge(srow, n, 1u, mx, T, red, &n_all);
    if (n_all == 0) return 0u;
    // ---- top-p: the shortest prefix of the sorted list whose probability reaches top_p
    uint32_t cut = 1u, cut_keep = 0xffffffffu;     // keys > cut are all kept, of the ties at `cut` the first cut_keep
    double kept = total;
    if (top_p < 1.0f) {
        const double target = (double)top_p * total;
        cut = smp_bisect(srow, n, target, false, mx, T, red);
        uint32_t c_ge = 0, c_gt = 0;
        const double m_ge = smp_mass_ge(srow, n, cut, mx, T, red, &c_ge);
        const double m_gt = cut == 0xffffffffu ? 0.0 : smp_mass_ge(srow, n, cut + 1u, mx, T, red, &c_gt);
        const uint32_t ties = c_ge - c_gt;
        const double e_tie = ties ? (m_ge - m_gt) / (double)ties : 0.0;
        uint32_t t = ties;
        if (e_tie > 0.0) {
            const double need = ceil((target - m_gt) / e_tie);
            t = need < 1.0 ? 1u : (need > (double)ties ? ties : (uint32_t)need);
        }
        cut_keep = t;
        kept = m_gt + (double)t * e_tie;
    }
    // ---- the draw: walk the kept prefix until the cumulative probability passes r
    const double R = r * kept;
    uint32_t phi = smp_bisect(srow, n, R, true, mx, T, red);
    if (phi < cut) phi = cut;                        // rounding pushed the walk past the prefix: its last element
    uint32_t c_ge = 0, c_gt = 0;
    const double m_ge = smp_mass_ge(srow, n, phi, mx, T, red, &c_ge);
    const double m_gt = phi == 0xffffffffu ? 0.0 : smp_mass_ge(srow, n, phi + 1u, mx, T, red, &c_gt);
    uint32_t ties = c_ge - c_gt;
    if (phi == cut && cut_keep < ties) ties = cut_keep;
    const double e_tie = (c_ge - c_gt) ? (m_ge - m_gt) / (double)(c_ge - c_gt) : 0.0;
    uint32_t t_idx = 0;
    if (e_tie > 0.0 && R > m_gt) {
        const double q = floor((R - m_gt) / e_tie);
        t_idx = q >= (double)ties ? ties - 1 : (uint32_t)q;
    }
    if (ties == 0) return 0u;
    // ---- the t_idx-th candidate (ascending id) whose key is phi: every thread counts a contiguous range of ids
    const uint32_t chunk = (n + SMP_THREADS - 1) / SMP_THREADS;
    const uint32_t lo = tid * chunk, hi = lo + chunk < n ? lo + chunk : n;
    uint32_t mine = 0;
    for (uint32_t i = lo; i < hi; i++) mine += (smp_key(srow[i]) == phi && srow[i] == srow[i]) ? 1u : 0u;
    __syncthreads();
    scan[tid] = mine;
    __syncthreads();
    uint32_t before = 0;
    for (uint32_t w = 0; w < tid; w++) before += scan[w];
    __syncthreads();
    if (t_idx >= before && t_idx < before + mine) {
        uint32_t k = t_idx - before;
        for (uint32_t i = lo; i < hi; i++)
            if (smp_key(srow[i]) == phi && srow[i] == srow[i]) {
                if (k == 0) { scan[SMP_THREADS] = i; break; }
                k--;
            }
    }
    __syncthreads();
    return scan[SMP_THREADS];
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_rows_kernel(const float* __restrict__ logits, uint32_t n, uint32_t ld, const uint32_t* __restrict__ seen,
                   const uint32_t* __restrict__ seen_off, float penalty, float temperature, uint32_t top_k, float top_p,
                   uint64_t seed, uint64_t step, const int32_t* __restrict__ row_active, uint32_t* __restrict__ out_idx) {
    extern __shared__ float srow[];                       // n logits, then the seen-id bitmap
    uint32_t* bits = reinterpret_cast<uint32_t*>(srow + n);
    __shared__ float wv[32];
    __shared__ uint32_t wi[32];
    __shared__ __align__(8) float cand_v[SMP_MAX_K];
    __shared__ uint32_t cand_i[SMP_MAX_K + 1];
    const uint32_t row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (row_active && row_active[row] < 0) return;
    const float* l = logits + (size_t)row * ld;
    const uint32_t nwords = (n + 31) / 32;
    for (uint32_t i = tid; i < nwords; i += SMP_THREADS) bits[i] = 0u;
    for (uint32_t i = tid; i < n; i += SMP_THREADS) srow[i] = l[i];
    __syncthreads();
    if (penalty != 1.0f && seen) {
        for (uint32_t i = seen_off[row] + tid; i < seen_off[row + 1]; i += SMP_THREADS) {
            uint32_t id = seen[i];
            if (id < n) atomicOr(&bits[id >> 5], 1u << (id & 31));
        }
        __syncthreads();
        for (uint32_t i = tid; i < n; i += SMP_THREADS)
            if (bits[i >> 5] & (1u << (i & 31))) srow[i] = srow[i] > 0.0f ? srow[i] / penalty : srow[i] * penalty;
        __syncthreads();
    }
    if (temperature > 0.0f && (top_k == 0 || top_k >= n)) {
        // no truncation: bisection over the whole row (the selection loop below only serves small k)
        double* red = reinterpret_cast<double*>(cand_v);          // 64 doubles
        const uint64_t bitsr = smp_mix(seed ^ smp_mix(step * 0x632BE59BD9B4E019ull + row + 1));
        const double r = (double)(bitsr >> 11) * (1.0 / 9007199254740992.0);
        const uint32_t pick = smp_sample_untruncated(srow, n, temperature, top_p, r, red, cand_i);
        if (tid == 0) out_idx[row] = pick;
        return;
    }
    const uint32_t k = (temperature <= 0.0f) ? 1u : top_k;
    for (uint32_t c = 0; c < k; c++) {
        float best = -INFINITY;
        uint32_t bi = 0xffffffffu;
        for (uint32_t i = tid; i < n; i += SMP_THREADS) {
            float v = srow[i];
            if (v > best || (v == best && i < bi)) { best = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_combine(best, bi, ov, oi);
        }
        if (lane == 0) { wv[warp] = best; wi[warp] = bi; }
        __syncthreads();
        if (warp == 0) {
            best = wv[lane];
            bi = wi[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, best, o);
                uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                argmax_combine(best, bi, ov, oi);
            }
            if (lane == 0) {
                cand_v[c] = best;
                cand_i[c] = bi;
                if (bi != 0xffffffffu) srow[bi] = -INFINITY;  // taken
            }
        }
        __syncthreads();
    }
    if (tid != 0) return;
    if (temperature <= 0.0f) { out_idx[row] = cand_i[0] == 0xffffffffu ? 0u : cand_i[0]; return; }
    // candidates that ran out (-inf everywhere) end the list
    uint32_t m = 0;
    while (m < k && cand_i[m] != 0xffffffffu) m++;
    if (m == 0) { out_idx[row] = 0; return; }
    // f64 softmax over the candidates, reusing srow as f64 scratch is not possible (taken marks):
    // k <= 1024 doubles are recomputed on the fly instead of stored.
    const double mx = (double)cand_v[0], T = (double)temperature;
    double sum = 0.0;
    for (uint32_t j = 0; j < m; j++) sum += exp(((double)cand_v[j] - mx) / T);
    uint32_t keep = m;
    if (top_p < 1.0f) {
        double cum = 0.0;
        for (uint32_t j = 0; j < m; j++) {
            cum += exp(((double)cand_v[j] - mx) / T) / sum;
            if (cum >= (double)top_p) { keep = j + 1; break; }
        }
    }
    double s2 = 0.0;
    for (uint32_t j = 0; j < keep; j++) s2 += exp(((double)cand_v[j] - mx) / T) / sum;
    const uint64_t bitsr = smp_mix(seed ^ smp_mix(step * 0x632BE59BD9B4E019ull + row + 1));
    double r = (double)(bitsr >> 11) * (1.0 / 9007199254740992.0);  // [0, 1)
    uint32_t pick = cand_i[keep - 1];
    for (uint32_t j = 0; j < keep; j++) {
        double p = (exp(((double)cand_v[j] - mx) / T) / sum) / s2;
        if (r < p) { pick = cand_i[j]; break; }
        r -= p;
    }
    out_idx[row] = pick;
}

int launch_sample_rows(cudaStream_t st, const float* logits, uint32_t rows, uint32_t n, uint32_t ld, const uint32_t* seen,
                       const uint32_t* seen_off, float penalty, float temperature, uint32_t top_k, float top_p, uint64_t seed,
                       uint64_t step, const int32_t* row_active, uint32_t* out_idx) {
    if (rows == 0 || n == 0) return AK_OK;
    AK_REQUIRE(temperature <= 0.0f || top_k <= SMP_MAX_K || top_k >= n, AK_ERR_UNSUPPORTED,
               "sampler: top_k must be 0 (no truncation) or 1..%d on the device (got %u)", SMP_MAX_K, top_k);
    const size_t smem = (size_t)n * 4 + (size_t)((n + 31) / 32) * 4;
    AK_REQUIRE(smem <= 214 * 1024, AK_ERR_UNSUPPORTED, "sampler: vocabulary of %u does not fit shared memory", n);
    AK_CUDA(cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    sample_rows_kernel<<<rows, SMP_THREADS, smem, st>>>(logits, n, ld, seen, seen_off, penalty, temperature, top_k, top_p, seed, step,
                                                        row_active, out_idx);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

}  // namespace ak

extern "C" int ak_sample_token(void* stream, const float* logits, uint32_t rows, uint32_t n, const uint32_t* seen,
                               const uint32_t* seen_off, float repetition_penalty, float temperature, uint32_t top_k, float top_p,
                               uint64_t seed, uint64_t step, uint32_t* out_idx) {
    AK_REQUIRE(logits && out_idx, AK_ERR_INVALID_ARG, "ak_sample_token: null pointer");
    AK_REQUIRE(repetition_penalty == 1.0f || (seen && seen_off), AK_ERR_INVALID_ARG, "ak_sample_token: a repetition penalty needs the seen ids");
    return ak::launch_sample_rows(ak::as_stream(stream), logits, rows, n, n, seen, seen_off, repetition_penalty, temperature, top_k,
                                  top_p, seed, step, nullptr, out_idx);
}
