// Causal prefill attention over ragged (varlen) sequences: the online-softmax recurrence of the
// reference's FLASH_ATTENTION kernel (src/shaders/cuda.rs:633-685: score*scale, running max,
// acc = acc*corr + p*v, final divide by the running sum), tiled 64 queries x 64 keys per CTA
// with fp32 accumulation. K/V come either from the paged pools through a block table (engine
// and session) or from contiguous [seq, dim] buffers (the reference emitter's form).
#include "kernels.h"

namespace ak {

constexpr int PF_BK = 64, PF_THREADS = 256, PF_BS = 16;

// RPT = query rows per thread: the query tile is 16*RPT rows. RPT = 4 (64-row tiles) has the best
// FMA-to-shared-load ratio; RPT = 1 (16-row tiles) makes four times as many CTAs, which is what a
// single short prompt joining a decode batch needs to occupy the machine.
template <typename T, int HD, int RPT> struct PfSmem {
    static constexpr int BQ = 16 * RPT;
    float qt[HD][BQ + 4];   // Q^T
    float kt[HD][PF_BK + 4];   // K^T
    float vs[PF_BK][HD + 4];   // V
    float pt[PF_BK][BQ + 4];  // P^T
};

template <typename T> __device__ __forceinline__ void load_chunk(const T* src, float* out);
template <> __device__ __forceinline__ void load_chunk<float>(const float* src, float* out) {
    float4 v = *reinterpret_cast<const float4*>(src);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <> __device__ __forceinline__ void load_chunk<bf16>(const bf16* src, float* out) {
    uint4 raw = *reinterpret_cast<const uint4*>(src);
    out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
    out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
    out[4] = __uint_as_float(raw.z << 16); out[5] = __uint_as_float(raw.z & 0xffff0000u);
    out[6] = __uint_as_float(raw.w << 16); out[7] = __uint_as_float(raw.w & 0xffff0000u);
}

// grid: (q tiles, heads, sequences). PAGED: k/v are pools + block table; else contiguous rows.
template <typename T, int HD, bool PAGED, int RPT>
__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_kernel(const T* __restrict__ q, const T* __restrict__ kbase, const T* __restrict__ vbase,
                    const int32_t* __restrict__ block_tables, uint32_t max_blocks, const int32_t* __restrict__ cu,
                    const int32_t* __restrict__ seq_slot, T* __restrict__ out, float* __restrict__ l_cache,
                    uint32_t row_base, uint32_t heads, float scale, uint32_t fixed_len) {
    pdl_wait();
    pdl_trigger();
    constexpr int EPC = 16 / (int)sizeof(T);
    constexpr int CPR = HD / EPC;      // 16-byte chunks per row
    constexpr int OC = HD / 16;        // output columns per thread
    extern __shared__ uint8_t smem_raw[];
    constexpr int PF_BQ = 16 * RPT;
    PfSmem<T, HD, RPT>& sm = *reinterpret_cast<PfSmem<T, HD, RPT>*>(smem_raw);

    const uint32_t seq = blockIdx.z, h = blockIdx.y, qtile = blockIdx.x;
    const uint32_t dim = heads * HD;
    uint32_t row0, len;
    if (cu) { row0 = row_base + (uint32_t)cu[seq]; len = (uint32_t)(cu[seq + 1] - cu[seq]); }
    else { row0 = row_base; len = fixed_len; }
    const uint32_t q0 = qtile * PF_BQ;
    if (q0 >= len) return;
    const int32_t* table = PAGED ? block_tables + (size_t)seq_slot[seq] * max_blocks : nullptr;
    const uint32_t tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

    // ---- Q tile -> qt (transposed). thread -> (row = e % 64, chunk = e / 64)
    for (uint32_t e = tid; e < PF_BQ * CPR; e += PF_THREADS) {
        uint32_t r = e % PF_BQ, c = e / PF_BQ;
        float v[EPC];
        if (q0 + r < len) load_chunk<T>(q + (size_t)(row0 + q0 + r) * dim + (size_t)h * HD + c * EPC, v);
        else
#pragma unroll
            for (int i = 0; i < EPC; i++) v[i] = 0.0f;
#pragma unroll
        for (int i = 0; i < EPC; i++) sm.qt[c * EPC + i][r] = v[i];
    }

    float m_run[RPT], l_run[RPT], o[RPT][OC];
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        m_run[i] = -INFINITY; l_run[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < OC; c++) o[i][c] = 0.0f;
    }

    const uint32_t q_last = (q0 + PF_BQ - 1 < len - 1) ? q0 + PF_BQ - 1 : len - 1;
    for (uint32_t k0 = 0; k0 <= q_last; k0 += PF_BK) {
        __syncthreads();  // previous tile fully consumed (also orders the Q store before first use)
        // ---- K tile -> kt (transposed), V tile -> vs
        for (uint32_t e = tid; e < PF_BK * CPR; e += PF_THREADS) {
            uint32_t r = e % PF_BK, c = e / PF_BK;
            uint32_t kj = k0 + r;
            float v[EPC];
            if (kj < len) {
                const T* src;
                if (PAGED) src = kbase + (((size_t)table[kj / PF_BS] * heads + h) * PF_BS + (kj % PF_BS)) * HD + c * EPC;
                else src = kbase + (size_t)(row0 + kj) * dim + (size_t)h * HD + c * EPC;
                load_chunk<T>(src, v);
            } else {
#pragma unroll
                for (int i = 0; i < EPC; i++) v[i] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < EPC; i++) sm.kt[c * EPC + i][r] = v[i];
        }
        for (uint32_t e = tid; e < PF_BK * CPR; e += PF_THREADS) {
            uint32_t c = e % CPR, r = e / CPR;
            uint32_t kj = k0 + r;
            float v[EPC];
            if (kj < len) {
                const T* src;
                if (PAGED) src = vbase + (((size_t)table[kj / PF_BS] * heads + h) * PF_BS + (kj % PF_BS)) * HD + c * EPC;
                else src = vbase + (size_t)(row0 + kj) * dim + (size_t)h * HD + c * EPC;
                load_chunk<T>(src, v);
            } else {
#pragma unroll
                for (int i = 0; i < EPC; i++) v[i] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < EPC; i++) sm.vs[r][c * EPC + i] = v[i];
        }
        __syncthreads();

        // ---- S = Q K^T for rows RPT*ty..RPT*ty+RPT-1, keys 4tx..4tx+3
        float s[RPT][4];
#pragma unroll
        for (int i = 0; i < RPT; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) s[i][j] = 0.0f;
#pragma unroll 8
        for (int d = 0; d < HD; d++) {
            float qa_[RPT];
#pragma unroll
            for (int i = 0; i < RPT; i++) qa_[i] = sm.qt[d][ty * RPT + i];
            float4 kb = *reinterpret_cast<const float4*>(&sm.kt[d][tx * 4]);
            float kb_[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int i = 0; i < RPT; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) s[i][j] = fmaf(qa_[i], kb_[j], s[i][j]);
        }
        // ---- mask, online softmax (16 lanes share a row group)
#pragma unroll
        for (int i = 0; i < RPT; i++) {
            uint32_t qi = q0 + ty * RPT + i;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t kj = k0 + tx * 4 + j;
                s[i][j] = (kj > qi || kj >= len) ? -INFINITY : s[i][j] * scale;
                mx = fmaxf(mx, s[i][j]);
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            float m_new = fmaxf(m_run[i], mx);
            float corr = (m_new == -INFINITY) ? 1.0f : expf(m_run[i] - m_new);
            float rs = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float pv = (s[i][j] == -INFINITY) ? 0.0f : expf(s[i][j] - m_new);
                s[i][j] = pv;
                rs += pv;
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, off);
            l_run[i] = l_run[i] * corr + rs;
            m_run[i] = m_new;
#pragma unroll
            for (int c = 0; c < OC; c++) o[i][c] *= corr;
        }
        // ---- P^T to shared
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int i = 0; i < RPT; i++) sm.pt[tx * 4 + j][ty * RPT + i] = s[i][j];
        __syncthreads();
        // ---- O += P V, thread owns rows 4ty..+3 and columns tx*OC..+OC-1
#pragma unroll 4
        for (int j = 0; j < PF_BK; j++) {
            float pa_[RPT];
#pragma unroll
            for (int i = 0; i < RPT; i++) pa_[i] = sm.pt[j][ty * RPT + i];
            float vv[OC];
#pragma unroll
            for (int c = 0; c < OC; c += 4) {
                float4 t = *reinterpret_cast<const float4*>(&sm.vs[j][tx * OC + c]);
                vv[c] = t.x; vv[c + 1] = t.y; vv[c + 2] = t.z; vv[c + 3] = t.w;
            }
#pragma unroll
            for (int i = 0; i < RPT; i++)
#pragma unroll
                for (int c = 0; c < OC; c++) o[i][c] = fmaf(pa_[i], vv[c], o[i][c]);
        }
    }
    // ---- write
#pragma unroll
    for (int i = 0; i < RPT; i++) {
        uint32_t qi = q0 + ty * RPT + i;
        if (qi >= len) continue;
        float inv = 1.0f / l_run[i];
        T* dst = out + (size_t)(row0 + qi) * dim + (size_t)h * HD + tx * OC;
#pragma unroll
        for (int c = 0; c < OC; c++) dst[c] = Cvt<T>::from_f(o[i][c] * inv);
        if (l_cache && tx == 0) l_cache[(size_t)qi * heads + h] = m_run[i] + logf(l_run[i]);
    }
}

// Any head_dim: one warp per (query row, head), keys striped over lanes, two passes through a
// shared score row. For the reference's small test shapes (head_dim 4, 8, 16); not a hot path.
template <typename T, bool PAGED>
__global__ void attn_prefill_generic_kernel(const T* __restrict__ q, const T* __restrict__ kbase,
                                            const T* __restrict__ vbase, const int32_t* __restrict__ block_tables,
                                            uint32_t max_blocks, const int32_t* __restrict__ cu,
                                            const int32_t* __restrict__ seq_slot, T* __restrict__ out,
                                            float* __restrict__ l_cache, uint32_t row_base, uint32_t heads, uint32_t hd,
                                            float scale, uint32_t fixed_len) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float sc[];  // (qi+1) scores
    const uint32_t seq = blockIdx.z, h = blockIdx.y, qi = blockIdx.x, lane = threadIdx.x;
    const uint32_t dim = heads * hd;
    uint32_t row0, len;
    if (cu) { row0 = row_base + (uint32_t)cu[seq]; len = (uint32_t)(cu[seq + 1] - cu[seq]); }
    else { row0 = row_base; len = fixed_len; }
    if (qi >= len) return;
    const int32_t* table = PAGED ? block_tables + (size_t)seq_slot[seq] * max_blocks : nullptr;
    const T* qr = q + (size_t)(row0 + qi) * dim + (size_t)h * hd;
    float mx = -INFINITY;
    for (uint32_t j = lane; j <= qi; j += 32) {
        const T* kr = PAGED ? kbase + (((size_t)table[j / PF_BS] * heads + h) * PF_BS + (j % PF_BS)) * hd
                            : kbase + (size_t)(row0 + j) * dim + (size_t)h * hd;
        float s = 0.0f;
        for (uint32_t c = 0; c < hd; c++) s = fmaf(Cvt<T>::to_f(qr[c]), Cvt<T>::to_f(kr[c]), s);
        s *= scale;
        sc[j] = s;
        mx = fmaxf(mx, s);
    }
    mx = warp_max(mx);
    float sum = 0.0f;
    for (uint32_t j = lane; j <= qi; j += 32) {
        float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (uint32_t d = lane; d < hd; d += 32) {
        float o = 0.0f;
        for (uint32_t j = 0; j <= qi; j++) {
            const T* vr = PAGED ? vbase + (((size_t)table[j / PF_BS] * heads + h) * PF_BS + (j % PF_BS)) * hd
                                : vbase + (size_t)(row0 + j) * dim + (size_t)h * hd;
            o = fmaf(sc[j], Cvt<T>::to_f(vr[d]), o);
        }
        out[(size_t)(row0 + qi) * dim + (size_t)h * hd + d] = Cvt<T>::from_f(o / sum);
    }
    if (l_cache && lane == 0) l_cache[(size_t)qi * heads + h] = mx + logf(sum);
}

template <typename T, int HD, bool PAGED, int RPT>
static int launch_tiled_rpt(cudaStream_t st, const T* q, const T* k, const T* v, const int32_t* bt, uint32_t max_blocks,
                            const int32_t* cu, const int32_t* seq_slot, T* out, float* l_cache, uint32_t n_seqs,
                            uint32_t max_len, uint32_t row_base, uint32_t heads, float scale, uint32_t fixed_len) {
    constexpr int PF_BQ = 16 * RPT;
    size_t smem = sizeof(PfSmem<T, HD, RPT>);
    static bool attr_set[64] = {};
    int dev = 0;
    AK_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(device_cache_mutex());
    if (!attr_set[dev & 63]) {
        AK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<T, HD, PAGED, RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev & 63] = true;
    }
    dim3 grid(cdiv(max_len, PF_BQ), heads, n_seqs);
    AK_TRY(launch_k(attn_prefill_kernel<T, HD, PAGED, RPT>, dim3(grid), dim3(PF_THREADS), smem, st, NO_CLUSTER, q, k, v, bt, max_blocks, cu, seq_slot, out, l_cache,
                                                                       row_base, heads, scale, fixed_len));
    return AK_OK;
}

template <typename T, int HD, bool PAGED>
static int launch_tiled(cudaStream_t st, const T* q, const T* k, const T* v, const int32_t* bt, uint32_t max_blocks,
                        const int32_t* cu, const int32_t* seq_slot, T* out, float* l_cache, uint32_t n_seqs,
                        uint32_t max_len, uint32_t row_base, uint32_t heads, float scale, uint32_t fixed_len) {
    // 64-row query tiles when they already give two waves of CTAs, else 16-row tiles
    const uint64_t big = (uint64_t)cdiv(max_len, 64) * heads * n_seqs;
    if (big >= 296)
        return launch_tiled_rpt<T, HD, PAGED, 4>(st, q, k, v, bt, max_blocks, cu, seq_slot, out, l_cache, n_seqs, max_len, row_base, heads, scale, fixed_len);
    return launch_tiled_rpt<T, HD, PAGED, 1>(st, q, k, v, bt, max_blocks, cu, seq_slot, out, l_cache, n_seqs, max_len, row_base, heads, scale, fixed_len);
}

template <typename T, bool PAGED>
static int launch_generic(cudaStream_t st, const T* q, const T* k, const T* v, const int32_t* bt, uint32_t max_blocks,
                          const int32_t* cu, const int32_t* seq_slot, T* out, float* l_cache, uint32_t n_seqs,
                          uint32_t max_len, uint32_t row_base, uint32_t heads, uint32_t hd, float scale, uint32_t fixed_len) {
    size_t smem = (size_t)max_len * sizeof(float);
    AK_REQUIRE(smem <= 200 * 1024, AK_ERR_UNSUPPORTED, "prefill attention (generic head_dim): sequence too long (%u)", max_len);
    if (smem > 48 * 1024)
        AK_CUDA(cudaFuncSetAttribute(attn_prefill_generic_kernel<T, PAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(max_len, heads, n_seqs);
    AK_TRY(launch_k(attn_prefill_generic_kernel<T, PAGED>, dim3(grid), dim3(32), smem, st, NO_CLUSTER, q, k, v, bt, max_blocks, cu, seq_slot, out, l_cache, row_base,
                                                                  heads, hd, scale, fixed_len));
    return AK_OK;
}

int launch_attn_prefill_paged(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                              const int32_t* block_tables, uint32_t max_blocks_per_seq, const int32_t* cu,
                              const int32_t* seq_slot, const int32_t* pos0, void* out, uint32_t n_seqs, uint32_t max_len, uint32_t row_base,
                              uint32_t heads, uint32_t head_dim, uint32_t block_size, float scale, uint32_t dtype,
                              uint64_t q_rows, uint64_t pool_blocks) {
    if (n_seqs == 0 || max_len == 0) return AK_OK;
    AK_REQUIRE(block_size == PF_BS, AK_ERR_UNSUPPORTED, "prefill attention: block_size must be 16");
    // bf16 with a tensor-core friendly head size: the tcgen05 kernel (needs the extents for its tensor maps)
    if (dtype == AK_BF16 && (head_dim == 64 || head_dim == 128) && q_rows && pool_blocks)
        return launch_attn_prefill_tc(st, q, q_rows, k_pool, v_pool, pool_blocks, block_tables, max_blocks_per_seq, cu, seq_slot, pos0, out,
                                      n_seqs, max_len, row_base, heads, head_dim, scale);
    if (dtype == AK_F32) {
        auto Q = (const float*)q; auto K = (const float*)k_pool; auto V = (const float*)v_pool; auto O = (float*)out;
        if (head_dim == 64) return launch_tiled<float, 64, true>(st, Q, K, V, block_tables, max_blocks_per_seq, cu, seq_slot, O, nullptr, n_seqs, max_len, row_base, heads, scale, 0);
        if (head_dim == 128) return launch_tiled<float, 128, true>(st, Q, K, V, block_tables, max_blocks_per_seq, cu, seq_slot, O, nullptr, n_seqs, max_len, row_base, heads, scale, 0);
        return launch_generic<float, true>(st, Q, K, V, block_tables, max_blocks_per_seq, cu, seq_slot, O, nullptr, n_seqs, max_len, row_base, heads, head_dim, scale, 0);
    }
    auto Q = (const bf16*)q; auto K = (const bf16*)k_pool; auto V = (const bf16*)v_pool; auto O = (bf16*)out;
    if (head_dim == 64) return launch_tiled<bf16, 64, true>(st, Q, K, V, block_tables, max_blocks_per_seq, cu, seq_slot, O, nullptr, n_seqs, max_len, row_base, heads, scale, 0);
    if (head_dim == 128) return launch_tiled<bf16, 128, true>(st, Q, K, V, block_tables, max_blocks_per_seq, cu, seq_slot, O, nullptr, n_seqs, max_len, row_base, heads, scale, 0);
    return launch_generic<bf16, true>(st, Q, K, V, block_tables, max_blocks_per_seq, cu, seq_slot, O, nullptr, n_seqs, max_len, row_base, heads, head_dim, scale, 0);
}

int launch_flash_attention_f32(cudaStream_t st, const float* q, const float* k, const float* v, float* out,
                               float* l_cache, ak_flash_attn_meta m) {
    if (m.seq_len == 0) return AK_OK;
    AK_REQUIRE(m.head_dim >= 1 && m.dim % m.head_dim == 0, AK_ERR_INVALID_ARG, "flash_attention: head_dim must divide dim");
    uint32_t heads = m.dim / m.head_dim;
    bool aligned = ((uintptr_t)q % 16 == 0) && ((uintptr_t)k % 16 == 0) && ((uintptr_t)v % 16 == 0);
    if (m.head_dim == 64 && aligned)
        return launch_tiled<float, 64, false>(st, q, k, v, nullptr, 0, nullptr, nullptr, out, l_cache, 1, m.seq_len, m.row_offset, heads, m.scale, m.seq_len);
    if (m.head_dim == 128 && aligned)
        return launch_tiled<float, 128, false>(st, q, k, v, nullptr, 0, nullptr, nullptr, out, l_cache, 1, m.seq_len, m.row_offset, heads, m.scale, m.seq_len);
    return launch_generic<float, false>(st, q, k, v, nullptr, 0, nullptr, nullptr, out, l_cache, 1, m.seq_len, m.row_offset, heads, m.head_dim, m.scale, m.seq_len);
}

}  // namespace ak

using namespace ak;
extern "C" int ak_flash_attention(void* stream, const float* q, const float* k, const float* v, float* out, float* l_cache,
                                  ak_flash_attn_meta m) {
    AK_REQUIRE(q && k && v && out, AK_ERR_INVALID_ARG, "ak_flash_attention: null pointer");
    return launch_flash_attention_f32(as_stream(stream), q, k, v, out, l_cache, m);
}

extern "C" int ak_attn_prefill_paged(void* stream, const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                                     uint32_t max_blocks_per_seq, const int32_t* cu, const int32_t* seq_slot, void* out, uint32_t n_seqs,
                                     uint32_t max_len, uint32_t q_rows, uint32_t heads, uint32_t head_dim, float scale, uint32_t dtype,
                                     uint32_t pool_blocks) {
    AK_REQUIRE(q && k_pool && v_pool && block_tables && cu && seq_slot && out, AK_ERR_INVALID_ARG, "ak_attn_prefill_paged: null pointer");
    AK_REQUIRE(dtype == AK_F32 || dtype == AK_BF16, AK_ERR_INVALID_ARG, "ak_attn_prefill_paged: dtype must be f32 or bf16");
    AK_REQUIRE(heads >= 1 && head_dim >= 1, AK_ERR_INVALID_ARG, "ak_attn_prefill_paged: empty head shape");
    return launch_attn_prefill_paged(as_stream(stream), q, k_pool, v_pool, block_tables, max_blocks_per_seq, cu, seq_slot, nullptr, out, n_seqs,
                                     max_len, 0, heads, head_dim, 16, scale, dtype, q_rows, pool_blocks);
}
