// Ragged paged decode attention (one query row per sequence), the HBM-bound kernel of batched
// decode. Fuses the reference's attn_qk_cached -> softmax_rect -> attn_av_cached
// (src/shaders/cuda.rs:349-419; src/nn/inference_graphs.rs:428-456).
//
// Data layout: K pool and V pool are [n_blocks, heads, 16, head_dim]; a (block, head) pair is a
// contiguous 16 x head_dim tile. One CTA = 4 warps works on one (sequence, head[, split]).
// Each warp runs its OWN pipeline over the KV blocks it owns (block index = warp mod 4):
//   lane 0 issues TMA tiled loads (128-byte swizzle, so the later shared-memory reads are
//   bank-conflict free) of the K and V tile into a STAGES-deep ring, completion on one mbarrier
//   per stage; the 32 lanes compute 16 scores (2 lanes per position), run the online softmax
//   with warp shuffles only, and accumulate P.V with each lane owning head_dim/32 outputs.
// No CTA-wide barrier sits in the loop; the four warps' (max, sum, acc) are merged once at the
// end, and with n_splits > 1 the per-split partials are merged by a second small kernel.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a code in a status word
// and unwinds.
#include "kernels.h"
#include "tma.h"

#include <stdlib.h>

namespace ak {

__device__ unsigned int g_attn_decode_status = 0;
// Set by the runner around its own launches (host side, per thread): see `early` in the kernel.
thread_local bool g_attn_early = false;

constexpr int DEC_WARPS = 4;
constexpr int DEC_BS = 16;  // positions per KV block

template <typename T, int HD, int ST> struct DecCfg {
    static constexpr int GROUPS = HD * (int)sizeof(T) / 128;   // 128-byte column groups per row
    static constexpr int EPC = 16 / (int)sizeof(T);            // elements per 16-byte chunk
    static constexpr int EPG = 128 / (int)sizeof(T);           // elements per column group
    static constexpr int QREGS = GROUPS * 4 * EPC;             // q values held per lane
    static constexpr int EPL = HD / 32;                        // output dims per lane
    static constexpr int TILE_BYTES = DEC_BS * HD * (int)sizeof(T);  // one K (or V) tile
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int STAGES = ST;   // ring depth per warp
    static constexpr int SMEM_BYTES = DEC_WARPS * STAGES * STAGE_BYTES + 1024;  // + alignment slack
};

// exp for the softmax: the accurate routine in the fp32 (parity) instantiation, the fast
// ex2-based one for bf16 data.
template <typename T> __device__ __forceinline__ float sm_exp(float x) {
    if constexpr (sizeof(T) == 4) return expf(x);
    else return __expf(x);
}

template <typename T> __device__ __forceinline__ void unpack16(const uint4& raw, float* out);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& raw, float* out) {
    out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
    out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void unpack16<bf16>(const uint4& raw, float* out) {
    // bf16 -> f32 is a 16-bit shift
    out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
    out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
    out[4] = __uint_as_float(raw.z << 16); out[5] = __uint_as_float(raw.z & 0xffff0000u);
    out[6] = __uint_as_float(raw.w << 16); out[7] = __uint_as_float(raw.w & 0xffff0000u);
}

template <typename T, int HD, int ST>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_paged_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const T* __restrict__ q, const int32_t* __restrict__ block_tables,
                         const int32_t* __restrict__ kv_lens, T* __restrict__ out, float* __restrict__ scratch,
                         uint32_t heads, uint32_t max_blocks, float scale, uint32_t n_splits, uint32_t early) {
    // `early` = the caller guarantees that the kernel launched just before this one wrote nothing of
    // the cache except each sequence's newest position (the engine's append kernel). Then:
    // Programmatic dependent launch: the descriptor arrays (lengths, block tables) and every KV
    // block except the one holding the newest position were written before the preceding kernel
    // started, so they are fetched BEFORE waiting for it; q and the newest block come after.
    pdl_trigger();
    using C = DecCfg<T, HD, ST>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[DEC_WARPS][C::STAGES];
    __shared__ float sm_m[DEC_WARPS], sm_l[DEC_WARPS];
    __shared__ float sm_acc[DEC_WARPS][HD];

    const uint32_t h = blockIdx.x, row = blockIdx.y, split = blockIdx.z;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int32_t kv_len = kv_lens[row];
    const uint32_t dim = heads * HD;

    // block range of this split
    const uint32_t nblk = kv_len > 0 ? ((uint32_t)kv_len + DEC_BS - 1) / DEC_BS : 0;
    const uint32_t bps = (nblk + n_splits - 1) / n_splits;
    const uint32_t b_begin = split * bps;
    const uint32_t b_end = (b_begin + bps < nblk) ? b_begin + bps : nblk;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* my_smem = smem + (size_t)warp * C::STAGES * C::STAGE_BYTES;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < C::STAGES; s++) mbar_init(&full_bar[warp][s], 1);
        mbar_fence_init();
    }
    __syncwarp();

    const uint32_t p = lane >> 1, hh = lane & 1;
    const int32_t* table = block_tables + (size_t)row * max_blocks;
    // blocks of this warp: b_begin + warp, + DEC_WARPS, ...
    const uint32_t first = b_begin + warp;
    const uint32_t nmine = (first < b_end) ? (b_end - first + DEC_WARPS - 1) / DEC_WARPS : 0;

    auto issue = [&](uint32_t i) {  // lane 0 only
        uint32_t s = i % C::STAGES;
        uint32_t blk = (uint32_t)table[first + i * DEC_WARPS];
        int32_t y = (int32_t)((blk * heads + h) * DEC_BS);
        uint8_t* kdst = my_smem + (size_t)s * C::STAGE_BYTES;
        uint8_t* vdst = kdst + C::TILE_BYTES;
        mbar_expect_tx(&full_bar[warp][s], C::STAGE_BYTES);
#pragma unroll
        for (int g = 0; g < C::GROUPS; g++) {
            tma_load_2d(kdst + g * (DEC_BS * 128), &tmK, g * C::EPG, y, &full_bar[warp][s]);
            tma_load_2d(vdst + g * (DEC_BS * 128), &tmV, g * C::EPG, y, &full_bar[warp][s]);
        }
    };

    // first ring of loads; the block that holds the newest position (written by the preceding
    // kernel) is held back until that kernel is known to be complete
    const uint32_t pre = nmine < (uint32_t)C::STAGES ? nmine : (uint32_t)C::STAGES;
    uint32_t deferred = 0xffffffffu;
    if (!early) pdl_wait();
    if (lane == 0) {
        for (uint32_t i = 0; i < pre; i++) {
            if (early && first + i * DEC_WARPS + 1 == nblk) deferred = i;
            else issue(i);
        }
    }
    pdl_wait();
    if (lane == 0 && deferred != 0xffffffffu) issue(deferred);

    // q slice of this lane: position pair-half hh = lane & 1 owns chunks [4hh, 4hh+4) of every group
    float qreg[C::QREGS];
    {
        const T* qrow = q + (size_t)row * dim + (size_t)h * HD;
#pragma unroll
        for (int g = 0; g < C::GROUPS; g++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint4 raw = *reinterpret_cast<const uint4*>(qrow + g * C::EPG + (4 * hh + c) * C::EPC);
                unpack16<T>(raw, &qreg[(g * 4 + c) * C::EPC]);
            }
    }

    float m_run = -INFINITY, l_run = 0.0f;
    float acc[C::EPL];
#pragma unroll
    for (int e = 0; e < C::EPL; e++) acc[e] = 0.0f;
    bool failed = false;

    for (uint32_t i = 0; i < nmine; i++) {
        const uint32_t s = i % C::STAGES;
        if (!mbar_wait(&full_bar[warp][s], (i / C::STAGES) & 1u)) {
            failed = true;
            break;
        }
        const uint8_t* ksm = my_smem + (size_t)s * C::STAGE_BYTES;
        const uint8_t* vsm = ksm + C::TILE_BYTES;
        const uint32_t blk_idx = first + i * DEC_WARPS;
        const int32_t n_valid_raw = kv_len - (int32_t)(blk_idx * DEC_BS);
        const uint32_t n_valid = n_valid_raw >= DEC_BS ? DEC_BS : (uint32_t)n_valid_raw;

        // ---- scores: position p, this lane's half of every 128-byte group
        float sc = 0.0f;
#pragma unroll
        for (int g = 0; g < C::GROUPS; g++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t chunk = (4 * hh + c) ^ (p & 7);
                uint4 raw = *reinterpret_cast<const uint4*>(ksm + g * (DEC_BS * 128) + p * 128 + chunk * 16);
                float kf[C::EPC];
                unpack16<T>(raw, kf);
#pragma unroll
                for (int e = 0; e < C::EPC; e++) sc = fmaf(qreg[(g * 4 + c) * C::EPC + e], kf[e], sc);
            }
        sc += __shfl_xor_sync(0xffffffffu, sc, 1);
        sc = (p < n_valid) ? sc * scale : -INFINITY;

        // ---- online softmax over the block's 16 positions (lane pairs hold equal values)
        float mb = sc;
#pragma unroll
        for (int o = 16; o > 1; o >>= 1) mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, o));
        const float m_new = fmaxf(m_run, mb);
        const float corr = sm_exp<T>(m_run - m_new);
        const float pj = sm_exp<T>(sc - m_new);  // exp(-inf) = 0 for masked positions
        float lb = pj;
#pragma unroll
        for (int o = 16; o > 1; o >>= 1) lb += __shfl_xor_sync(0xffffffffu, lb, o);
        l_run = l_run * corr + lb;
        m_run = m_new;
#pragma unroll
        for (int e = 0; e < C::EPL; e++) acc[e] *= corr;

        // ---- P.V: lane owns dims [lane*EPL, lane*EPL+EPL)
        {
            constexpr int LB = C::EPL * (int)sizeof(T);  // bytes per lane per row (4, 8 or 16)
            const uint32_t byte_off = lane * LB;
            const uint32_t g = byte_off >> 7, cin = (byte_off & 127) >> 4, within = byte_off & 15;
            const uint8_t* vbase = vsm + g * (DEC_BS * 128) + within;
#pragma unroll
            for (int j = 0; j < DEC_BS; j++) {
                const float pw = __shfl_sync(0xffffffffu, pj, 2 * j);
                if ((uint32_t)j < n_valid) {
                    const uint8_t* vp = vbase + j * 128 + ((cin ^ (j & 7)) << 4);
                    if constexpr (LB == 4) {
                        uint32_t raw = *reinterpret_cast<const uint32_t*>(vp);
                        acc[0] = fmaf(pw, __uint_as_float(raw << 16), acc[0]);
                        acc[1] = fmaf(pw, __uint_as_float(raw & 0xffff0000u), acc[1]);
                    } else if constexpr (LB == 8 && sizeof(T) == 2) {
                        uint2 raw = *reinterpret_cast<const uint2*>(vp);
                        acc[0] = fmaf(pw, __uint_as_float(raw.x << 16), acc[0]);
                        acc[1] = fmaf(pw, __uint_as_float(raw.x & 0xffff0000u), acc[1]);
                        acc[2] = fmaf(pw, __uint_as_float(raw.y << 16), acc[2]);
                        acc[3] = fmaf(pw, __uint_as_float(raw.y & 0xffff0000u), acc[3]);
                    } else if constexpr (LB == 8) {
                        float2 v = *reinterpret_cast<const float2*>(vp);
                        acc[0] = fmaf(pw, v.x, acc[0]);
                        acc[1] = fmaf(pw, v.y, acc[1]);
                    } else {
                        float4 v = *reinterpret_cast<const float4*>(vp);
                        acc[0] = fmaf(pw, v.x, acc[0]);
                        acc[1] = fmaf(pw, v.y, acc[1]);
                        acc[2] = fmaf(pw, v.z, acc[2]);
                        acc[3] = fmaf(pw, v.w, acc[3]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0 && i + C::STAGES < nmine) issue(i + C::STAGES);
    }
    if (failed) {
        if (lane == 0) atomicExch(&g_attn_decode_status, 1u);
        // give the copies still in flight one more bounded chance to land before leaving
        for (uint32_t i2 = 0; i2 < (uint32_t)C::STAGES; i2++) (void)mbar_wait(&full_bar[warp][i2], 0);
    }

    // ---- merge the four warps
    if (lane == 0) { sm_m[warp] = m_run; sm_l[warp] = l_run; }
#pragma unroll
    for (int e = 0; e < C::EPL; e++) sm_acc[warp][lane * C::EPL + e] = acc[e];
    __syncthreads();
    if (warp == 0) {
        float M = sm_m[0];
#pragma unroll
        for (int w = 1; w < DEC_WARPS; w++) M = fmaxf(M, sm_m[w]);
        float L = 0.0f, o[C::EPL];
#pragma unroll
        for (int e = 0; e < C::EPL; e++) o[e] = 0.0f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < DEC_WARPS; w++) {
                float f = sm_exp<T>(sm_m[w] - M);
                L += sm_l[w] * f;
#pragma unroll
                for (int e = 0; e < C::EPL; e++) o[e] = fmaf(sm_acc[w][lane * C::EPL + e], f, o[e]);
            }
        }
        if (n_splits == 1) {
            float inv = (L > 0.0f) ? 1.0f / L : 0.0f;
            T* orow = out + (size_t)row * dim + (size_t)h * HD + lane * C::EPL;
#pragma unroll
            for (int e = 0; e < C::EPL; e++) orow[e] = Cvt<T>::from_f(o[e] * inv);
        } else {
            float* pr = scratch + (((size_t)row * heads + h) * n_splits + split) * (HD + 2);
            if (lane == 0) { pr[0] = M; pr[1] = L; }
#pragma unroll
            for (int e = 0; e < C::EPL; e++) pr[2 + lane * C::EPL + e] = o[e];
        }
    }
}

// Merge of split partials: grid (heads, rows), one warp.
template <typename T, int HD>
__global__ void attn_decode_combine_kernel(const float* __restrict__ scratch, T* __restrict__ out, uint32_t heads,
                                           uint32_t n_splits) {
    pdl_wait();
    pdl_trigger();
    constexpr int EPL = HD / 32;
    const uint32_t h = blockIdx.x, row = blockIdx.y, lane = threadIdx.x;
    const float* base = scratch + ((size_t)row * heads + h) * n_splits * (HD + 2);
    float M = -INFINITY;
    for (uint32_t s = 0; s < n_splits; s++) M = fmaxf(M, base[(size_t)s * (HD + 2)]);
    float L = 0.0f, o[EPL];
#pragma unroll
    for (int e = 0; e < EPL; e++) o[e] = 0.0f;
    if (M > -INFINITY) {
        for (uint32_t s = 0; s < n_splits; s++) {
            const float* pr = base + (size_t)s * (HD + 2);
            float f = sm_exp<T>(pr[0] - M);
            L += pr[1] * f;
#pragma unroll
            for (int e = 0; e < EPL; e++) o[e] = fmaf(pr[2 + lane * EPL + e], f, o[e]);
        }
    }
    float inv = (L > 0.0f) ? 1.0f / L : 0.0f;
    T* orow = out + ((size_t)row * heads + h) * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; e++) orow[e] = Cvt<T>::from_f(o[e] * inv);
}

// Any head_dim <= 256 (the reference's small test shapes use 4, 8 and 16): one CTA per
// (head, row), plain loads, scores staged in shared memory. Not a hot path.
template <typename T>
__global__ void attn_decode_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                           const T* __restrict__ v_pool, const int32_t* __restrict__ block_tables,
                                           const int32_t* __restrict__ kv_lens, T* __restrict__ out, uint32_t heads,
                                           uint32_t hd, uint32_t bs, uint32_t max_blocks, float scale) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float sc[];  // kv_len scores
    __shared__ float red[32];
    const uint32_t h = blockIdx.x, row = blockIdx.y;
    const int32_t len = kv_lens[row];
    const uint32_t dim = heads * hd;
    T* orow = out + (size_t)row * dim + (size_t)h * hd;
    if (len <= 0) {
        for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) orow[d] = Cvt<T>::from_f(0.0f);
        return;
    }
    const int32_t* table = block_tables + (size_t)row * max_blocks;
    const T* qh = q + (size_t)row * dim + (size_t)h * hd;
    float mx = -INFINITY;
    for (int32_t j = threadIdx.x; j < len; j += blockDim.x) {
        const T* kr = k_pool + (((size_t)table[j / bs] * heads + h) * bs + (j % bs)) * hd;
        float s = 0.0f;
        for (uint32_t c = 0; c < hd; c++) s = fmaf(Cvt<T>::to_f(qh[c]), Cvt<T>::to_f(kr[c]), s);
        s *= scale;
        sc[j] = s;
        mx = fmaxf(mx, s);
    }
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (uint32_t w = 1; w < nw; w++) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.0f;
    for (int32_t j = threadIdx.x; j < len; j += blockDim.x) {
        float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = 0.0f;
    for (uint32_t w = 0; w < nw; w++) sum += red[w];
    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.0f;
        for (int32_t j = 0; j < len; j++) {
            const T* vr = v_pool + (((size_t)table[j / bs] * heads + h) * bs + (j % bs)) * hd;
            o = fmaf(sc[j] / sum, Cvt<T>::to_f(vr[d]), o);
        }
        orow[d] = Cvt<T>::from_f(o);
    }
}

size_t attn_decode_scratch_bytes(uint32_t rows, uint32_t heads, uint32_t head_dim, uint32_t n_splits) {
    if (n_splits <= 1) return 0;
    return (size_t)rows * heads * n_splits * (head_dim + 2) * sizeof(float);
}

uint32_t attn_decode_pick_splits(uint32_t rows, uint32_t heads, uint32_t max_kv_len) {
    // Enough CTAs to fill 148 SMs x 3 resident CTAs, but never less than 4 KV blocks per split.
    uint64_t items = (uint64_t)rows * heads;
    if (items == 0) return 1;
    uint32_t want = (uint32_t)((444 + items - 1) / items);
    uint32_t cap = max_kv_len / (4 * DEC_BS);
    if (cap < 1) cap = 1;
    if (want > cap) want = cap;
    if (want > 32) want = 32;
    return want < 1 ? 1 : want;
}

template <typename T, int HD, int ST>
static int launch_fast_st(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                       const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                       const ak_attn_decode_params& p, uint32_t n_splits, uint64_t pool_rows) {
    using C = DecCfg<T, HD, ST>;
    CUtensorMap tmK, tmV;
    int rc = make_tmap_2d(&tmK, k_pool, sizeof(T), HD, pool_rows, (uint64_t)HD * sizeof(T), C::EPG, DEC_BS, TMA_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&tmV, v_pool, sizeof(T), HD, pool_rows, (uint64_t)HD * sizeof(T), C::EPG, DEC_BS, TMA_SWIZZLE_128B);
    if (rc) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    AK_CUDA(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        AK_CUDA(cudaFuncSetAttribute(attn_decode_paged_kernel<T, HD, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        attr_set[dev & 63] = true;
    }
    dim3 grid(p.heads, p.rows, n_splits);
    AK_TRY(launch_k(attn_decode_paged_kernel<T, HD, ST>, dim3(grid), dim3(DEC_WARPS * 32), C::SMEM_BYTES, st, NO_CLUSTER, 
        tmK, tmV, (const T*)q, block_tables, kv_lens, (T*)out, (float*)scratch, p.heads, p.max_blocks_per_seq, p.scale, n_splits, (uint32_t)(g_attn_early ? 1 : 0)));
    if (n_splits > 1) {
        dim3 g2(p.heads, p.rows);
        AK_TRY(launch_k(attn_decode_combine_kernel<T, HD>, dim3(g2), dim3(32), 0, st, NO_CLUSTER, (const float*)scratch, (T*)out, p.heads, n_splits));
    }
    return AK_OK;
}

// Ring depth: a 2-deep ring per warp keeps a CTA at 33 KB (bf16, head_dim 64), so 6 CTAs = 24
// warps share an SM and a 64-sequence decode batch is resident in ONE wave. More resident warps
// hide latency better than a deeper ring per warp. AK_ATTN_STAGES overrides (tuning).
template <typename T, int HD>
static int launch_fast(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                       const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                       const ak_attn_decode_params& p, uint32_t n_splits, uint64_t pool_rows) {
    constexpr int STAGE_BYTES = 2 * DEC_BS * HD * (int)sizeof(T);
    constexpr int DEEP = (STAGE_BYTES <= 4096) ? 4 : (STAGE_BYTES <= 8192 ? 3 : 2);
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("AK_ATTN_STAGES");
        forced = e ? atoi(e) : 0;
    }
    int want = 2;  // measured: 6 CTAs/SM x 2 stages beats 3 CTAs/SM x 4 stages at 64 and at 1024 sequences
    if (forced == 2 || forced == DEEP) want = forced;
    if (want == 2) return launch_fast_st<T, HD, 2>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, pool_rows);
    return launch_fast_st<T, HD, DEEP>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, pool_rows);
}

// Rows of the 2-D view [n_blocks*heads*16, head_dim] of a pool. With pool_blocks given, a block
// id outside the pool reads zeros (TMA out-of-range fill) instead of touching foreign memory.
static uint64_t pool_rows_bound(const ak_attn_decode_params& p) {
    if (p.pool_blocks) return (uint64_t)p.pool_blocks * p.heads * DEC_BS;
    return (uint64_t)1 << 31;
}

int launch_attn_decode_paged(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                             const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                             const ak_attn_decode_params& p) {
    if (p.rows == 0 || p.heads == 0) return AK_OK;
    AK_REQUIRE(p.block_size == DEC_BS, AK_ERR_UNSUPPORTED, "attn_decode_paged: block_size must be 16");
    AK_REQUIRE(p.kv_dtype <= AK_BF16, AK_ERR_INVALID_ARG, "attn_decode_paged: bad kv_dtype");
    const bool fast = (p.head_dim == 64 || p.head_dim == 128) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) &&
                      ((uintptr_t)q % 16 == 0);
    if (!fast) {
        AK_REQUIRE(p.head_dim >= 1 && p.head_dim <= 256, AK_ERR_UNSUPPORTED, "attn_decode_paged: head_dim must be 1..256");
        size_t smem = (size_t)p.max_blocks_per_seq * DEC_BS * sizeof(float);
        AK_REQUIRE(smem <= 200 * 1024, AK_ERR_UNSUPPORTED, "attn_decode_paged: generic path supports up to 51200 positions");
        dim3 grid(p.heads, p.rows);
        if (p.kv_dtype == AK_F32) {
            if (smem > 48 * 1024) AK_CUDA(cudaFuncSetAttribute(attn_decode_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            AK_TRY(launch_k(attn_decode_generic_kernel<float>, dim3(grid), dim3(128), smem, st, NO_CLUSTER, (const float*)q, (const float*)k_pool, (const float*)v_pool, block_tables, kv_lens,
                                                                       (float*)out, p.heads, p.head_dim, p.block_size, p.max_blocks_per_seq, p.scale));
        } else {
            if (smem > 48 * 1024) AK_CUDA(cudaFuncSetAttribute(attn_decode_generic_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            AK_TRY(launch_k(attn_decode_generic_kernel<bf16>, dim3(grid), dim3(128), smem, st, NO_CLUSTER, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_tables, kv_lens,
                                                                      (bf16*)out, p.heads, p.head_dim, p.block_size, p.max_blocks_per_seq, p.scale));
        }
        return AK_OK;
    }
    uint32_t n_splits = p.n_splits ? p.n_splits : attn_decode_pick_splits(p.rows, p.heads, p.max_blocks_per_seq * DEC_BS);
    AK_REQUIRE(n_splits == 1 || scratch, AK_ERR_INVALID_ARG, "attn_decode_paged: scratch required when n_splits > 1");
    const uint64_t rows_bound = pool_rows_bound(p);
    if (p.kv_dtype == AK_F32) {
        if (p.head_dim == 64) return launch_fast<float, 64>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, rows_bound);
        return launch_fast<float, 128>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, rows_bound);
    }
    if (p.head_dim == 64) return launch_fast<bf16, 64>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, rows_bound);
    return launch_fast<bf16, 128>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, rows_bound);
}

int attn_decode_status(unsigned int* out) {
    AK_CUDA(cudaMemcpyFromSymbol(out, g_attn_decode_status, sizeof(unsigned int)));
    return AK_OK;
}

}  // namespace ak

using namespace ak;
extern "C" {
size_t ak_attn_decode_scratch_bytes(const ak_attn_decode_params* p) {
    if (!p) return 0;
    uint32_t ns = p->n_splits ? p->n_splits : attn_decode_pick_splits(p->rows, p->heads, p->max_blocks_per_seq * DEC_BS);
    return attn_decode_scratch_bytes(p->rows, p->heads, p->head_dim, ns);
}
int ak_attn_decode_paged(void* stream, const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                         const int32_t* kv_lens, void* out, void* scratch, ak_attn_decode_params p) {
    AK_REQUIRE(q && k_pool && v_pool && block_tables && kv_lens && out, AK_ERR_INVALID_ARG, "ak_attn_decode_paged: null pointer");
    return launch_attn_decode_paged(as_stream(stream), q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p);
}
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of the split-KV decode attention.
//
// Some hosts may not allocate device memory at the moment they need attention: a plugin running
// inside somebody else's memory pool, a real-time loop that forbids allocator calls after start-up,
// or code running where the process has already handed all free HBM to a KV pool. For them the
// split-KV partials live in a fixed buffer that is part of the loaded library image, so the call
// needs no workspace from the caller and performs no cudaMalloc / cudaFree.
//
// The buffer is a file-scope __device__ array: every GPU that loads this library holds
// AK_NOALLOC_SCRATCH_BYTES of it until the process exits. In host code the array's NAME is only
// a host-side handle, not a device address, so the address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that pointer is what the kernels receive.
namespace ak {
constexpr size_t AK_NOALLOC_SCRATCH_BYTES = 8u << 20;  // 8 MiB of partials
static __device__ __align__(256) unsigned char g_noalloc_scratch[AK_NOALLOC_SCRATCH_BYTES];

static int noalloc_scratch_ptr(void** out) {
    static void* ptrs[64] = {};
    int dev = 0;
    AK_CUDA(cudaGetDevice(&dev));
    AK_REQUIRE(dev >= 0 && dev < 64, AK_ERR_UNSUPPORTED, "attn_decode_paged_noalloc: device index %d not supported", dev);
    if (!ptrs[dev]) {
        void* p = nullptr;
        AK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        AK_REQUIRE(p != nullptr, AK_ERR_CUDA, "attn_decode_paged_noalloc: symbol address lookup returned null");
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return AK_OK;
}
}  // namespace ak

extern "C" {
size_t ak_attn_decode_noalloc_max_scratch_bytes(void) { return AK_NOALLOC_SCRATCH_BYTES; }

int ak_attn_decode_paged_noalloc(void* stream, const void* q, const void* k_pool, const void* v_pool,
                                 const int32_t* block_tables, const int32_t* kv_lens, void* out, ak_attn_decode_params p) {
    AK_REQUIRE(q && k_pool && v_pool && block_tables && kv_lens && out, AK_ERR_INVALID_ARG, "ak_attn_decode_paged_noalloc: null pointer");
    const uint32_t ns = p.n_splits ? p.n_splits : attn_decode_pick_splits(p.rows, p.heads, p.max_blocks_per_seq * DEC_BS);
    const size_t need = attn_decode_scratch_bytes(p.rows, p.heads, p.head_dim, ns);
    AK_REQUIRE(need <= AK_NOALLOC_SCRATCH_BYTES, AK_ERR_UNSUPPORTED,
               "ak_attn_decode_paged_noalloc: rows*heads*n_splits*(head_dim+2)*4 = %zu bytes of split partials exceed the built-in "
               "%zu-byte buffer; lower n_splits or use ak_attn_decode_paged with caller scratch",
               need, (size_t)AK_NOALLOC_SCRATCH_BYTES);
    void* scratch = nullptr;
    int rc = noalloc_scratch_ptr(&scratch);
    if (rc) return rc;
    p.n_splits = ns;
    // Every partial the merge kernel reads is written by the split kernel of the same call, so the
    // buffer's previous contents never matter and nothing has to be cleared.
    return launch_attn_decode_paged(as_stream(stream), q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p);
}
}
