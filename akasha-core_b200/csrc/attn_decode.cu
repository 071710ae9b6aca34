// Ragged paged decode attention (one query row per sequence), the HBM-bound kernel of batched
// decode. Fuses the reference's attn_qk_cached -> softmax_rect -> attn_av_cached
// (src/shaders/cuda.rs:349-419; src/nn/inference_graphs.rs:428-456).
//
// Data layout: K pool and V pool are [n_blocks, heads, 16, head_dim]; a (block, head) pair is a
// contiguous 16 x head_dim tile. One CTA = 4 warps works on one (sequence, head, split): a
// sequence's KV blocks are divided evenly over up to n_splits CTAs (never fewer than 4 blocks per
// CTA), so that the longest sequence of a small batch is spread over several SMs.
// Each warp runs its OWN pipeline over the KV blocks it owns (block index = warp mod 4):
//   TMA tiled loads (128-byte swizzle, so the later shared-memory reads are bank-conflict free) of
//   the K and V tile into a STAGES-deep ring, completion on one mbarrier per stage. (Requesting the
//   blocks beyond the ring into L2 up front with TMA prefetches was measured and is slower: 19.2 us
//   against 16.1 us at 64 sequences.) The online softmax is warp-shuffle only.
//   bf16 pools: the 16 scores of a tile and P.V go through mma.sync.m16n8k16 (fragments read with
//   ldmatrix from the swizzled tiles; the query fills every row of the A operand, so the score
//   accumulators are already laid out as the A operand of P.V): ~80 instructions per warp and tile
//   where scalar code needs ~500, which is what kept the scalar kernel off the HBM roofline.
//   f32 pools (parity mode): scalar fp32 FMAs, 2 lanes per position.
// No CTA-wide barrier sits in the loop; the four warps' (max, sum, acc) are merged once at the end.
// With more than one split the CTA writes its partial to scratch and bumps an arrival counter; the
// CTA that arrives last merges the partials in split order (so the sum does not depend on who is
// last) and clears the counter: one launch, no second kernel, no waiting on other CTAs.
//
// Fused form (the engine's decode rows): the kernel also does the reference's head split, RoPE and cache
// append of the step's new token (head_gather x3 -> rope_offset x2 -> cache_write x2,
// src/nn/inference_graphs.rs:385-426). Every warp rotates its own copy of the query straight from the qkv
// projection's f32 output; the warp that owns the sequence's last KV block rotates the new key, stores the new
// key and value rows to the pools and patches them into its shared-memory copy of that block. One launch less
// per layer, and, as the preceding kernel (the qkv projection) never touches the cache, EVERY K/V tile is
// requested before the programmatic-dependent-launch wait: the HBM stream overlaps the projection's tail.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a code in a status word
// and unwinds.
#include "kernels.h"
#include "tma.h"

#include <algorithm>
#include <vector>

namespace ak {

__device__ unsigned int g_attn_decode_status = 0;
// Set by the runner around its own launches (host side, per thread): see `early` in the kernel.
thread_local bool g_attn_early = false;

constexpr int DEC_WARPS = 4;
constexpr int DEC_BS = 16;          // positions per KV block
constexpr int DEC_MIN_BLOCKS = 4;   // a split never gets fewer KV blocks than this (one per warp)
constexpr int DEC_MAX_SPLITS = 32;

template <typename T, int HD, int ST> struct DecCfg {
    static constexpr int GROUPS = HD * (int)sizeof(T) / 128;   // 128-byte column groups per row
    static constexpr int EPC = 16 / (int)sizeof(T);            // elements per 16-byte chunk
    static constexpr int EPG = 128 / (int)sizeof(T);           // elements per column group
    static constexpr int QREGS = GROUPS * 4 * EPC;             // q values held per lane (scalar path)
    static constexpr int EPL = HD / 32;                        // output dims per lane
    static constexpr int TILE_BYTES = DEC_BS * HD * (int)sizeof(T);  // one K (or V) tile
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int STAGES = ST;   // ring depth per warp
    static constexpr int SMEM_BYTES = DEC_WARPS * STAGES * STAGE_BYTES + 1024;  // + alignment slack
};

// exp for the softmax: the accurate routine in the fp32 (parity) instantiation; the bf16 kernel works
// in the base-2 domain (scores pre-multiplied by log2 e) with the ex2 unit.
template <typename T> __device__ __forceinline__ float sm_exp(float x) {
    if constexpr (sizeof(T) == 4) return expf(x);
    else return exp2f(x);
}
__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
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

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    bf162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Fused split + RoPE + append (see the top of the file). qkv == nullptr: plain attention over q.
struct DecFused {
    // Optional launch order of the rows: CTA (h, y) works on row row_order[y]. A permutation only moves work between
    // CTAs (hence between SMs); the engine uses it to give every SM a similar number of KV bytes.
    const int32_t* row_order;
    const float* qkv;       // [rows, 3 * heads * HD] f32: q | k | v of the step's new token of every sequence
    const float2* rope;     // [rope_len][HD / 2] (cos, sin)
    uint32_t rope_len;
    void* k_pool;           // the pools as plain pointers, for the append stores
    void* v_pool;
};

// How a sequence of nblk KV blocks is divided: n_act CTAs (<= n_splits) of bps blocks each, every one
// of them non-empty. A function of the sequence's own length only.
__device__ __forceinline__ void split_plan(uint32_t nblk, uint32_t n_splits, uint32_t& n_act, uint32_t& bps) {
    n_act = (nblk + DEC_MIN_BLOCKS - 1) / DEC_MIN_BLOCKS;
    if (n_act > n_splits) n_act = n_splits;
    if (n_act < 1) n_act = 1;
    bps = (nblk + n_act - 1) / n_act;
    if (bps) n_act = (nblk + bps - 1) / bps;
    if (n_act < 1) n_act = 1;
}

// Scratch layout: [rows*heads*n_splits] partials of (HD + 2) floats (max, sum, acc[HD]), then
// [rows*heads] arrival counters (uint32, zero between launches).
__host__ __device__ __forceinline__ size_t partial_floats(uint32_t rows, uint32_t heads, uint32_t hd, uint32_t n_splits) {
    return (size_t)rows * heads * n_splits * (hd + 2);
}

// Tail of both kernels, executed by warp 0 with this CTA's merged (M, L, o[EPL] per lane).
// Single split: normalise and store. Otherwise publish the partial; the last CTA to arrive for this
// (row, head) merges all n_act partials in split order and clears the counter for the next launch.
template <typename T, int HD>
__device__ __forceinline__ void finish_row(float M, float L, float (&o)[HD / 32], T* __restrict__ out, float* __restrict__ scratch,
                                           uint32_t row, uint32_t h, uint32_t heads, uint32_t rows, uint32_t split, uint32_t n_splits,
                                           uint32_t n_act, uint32_t lane) {
    constexpr int EPL = HD / 32;
    T* orow = out + ((size_t)row * heads + h) * HD + lane * EPL;
    if (n_act == 1) {
        const float inv = (L > 0.0f) ? 1.0f / L : 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; e++) orow[e] = Cvt<T>::from_f(o[e] * inv);
        return;
    }
    float* base = scratch + ((size_t)row * heads + h) * n_splits * (HD + 2);
    float* pr = base + (size_t)split * (HD + 2);
    if (lane == 0) { pr[0] = M; pr[1] = L; }
#pragma unroll
    for (int e = 0; e < EPL; e++) pr[2 + lane * EPL + e] = o[e];
    __threadfence();
    __syncwarp();
    unsigned int* counter = reinterpret_cast<unsigned int*>(scratch + partial_floats(rows, heads, HD, n_splits)) + (size_t)row * heads + h;
    unsigned int prev = 0;
    if (lane == 0) prev = atomicAdd(counter, 1u);
    prev = __shfl_sync(0xffffffffu, prev, 0);
    if (prev + 1 != n_act) return;
    __threadfence();
    float Mx = -INFINITY;
    for (uint32_t s = 0; s < n_act; s++) Mx = fmaxf(Mx, __ldcg(base + (size_t)s * (HD + 2)));
    float Ls = 0.0f, acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; e++) acc[e] = 0.0f;
    if (Mx > -INFINITY) {
        for (uint32_t s = 0; s < n_act; s++) {
            const float* ps = base + (size_t)s * (HD + 2);
            const float f = sm_exp<T>(__ldcg(ps) - Mx);
            Ls += __ldcg(ps + 1) * f;
#pragma unroll
            for (int e = 0; e < EPL; e++) acc[e] = fmaf(__ldcg(ps + 2 + lane * EPL + e), f, acc[e]);
        }
    }
    const float inv = (Ls > 0.0f) ? 1.0f / Ls : 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; e++) orow[e] = Cvt<T>::from_f(acc[e] * inv);
    if (lane == 0) *counter = 0u;
}

// Resident CTAs per SM the register budget must allow: with a 2-deep ring a CTA holds 33 KB (bf16, head_dim 64),
// so shared memory admits 6, and 6 x 148 = 888 slots take a 64-sequence x 12-head batch in ONE wave.
template <typename T, int HD, int ST> struct DecOcc {
    static constexpr int SMEM = DecCfg<T, HD, ST>::SMEM_BYTES + 2048;
    static constexpr int BY_SMEM = (227 * 1024) / SMEM;
    static constexpr int VALUE = BY_SMEM > 6 ? 6 : (BY_SMEM < 1 ? 1 : BY_SMEM);
};

template <typename T, int HD, int ST>
__global__ void __launch_bounds__(DEC_WARPS * 32, DecOcc<T, HD, ST>::VALUE)
attn_decode_paged_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const T* __restrict__ q, const int32_t* __restrict__ block_tables,
                         const int32_t* __restrict__ kv_lens, T* __restrict__ out, float* __restrict__ scratch,
                         uint32_t heads, uint32_t max_blocks, float scale, uint32_t n_splits, uint32_t early,
                         const DecFused fz) {
    // `early` = the caller guarantees that the kernel launched just before this one wrote nothing of
    // the cache except each sequence's newest position (the engine's append kernel; in the fused form
    // nothing of the cache at all), and nothing of the descriptor arrays. Then, under programmatic
    // dependent launch, the lengths, the block tables and every KV block except one the predecessor may
    // have written are fetched BEFORE waiting for that kernel; q (or qkv) comes after. Without `early`
    // nothing is read before the wait.
    pdl_trigger();
    if (!early) pdl_wait();
    const bool fused = fz.qkv != nullptr;
    if (threadIdx.x == 0) { tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); }
    using C = DecCfg<T, HD, ST>;
    constexpr bool MMA = (sizeof(T) == 2);
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[DEC_WARPS][C::STAGES];
    __shared__ float sm_m[DEC_WARPS], sm_l[DEC_WARPS];
    __shared__ float sm_acc[DEC_WARPS][HD];

    const uint32_t h = blockIdx.x, split = blockIdx.z;
    const uint32_t row = fz.row_order ? (uint32_t)fz.row_order[blockIdx.y] : blockIdx.y;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int32_t* table = block_tables + (size_t)row * max_blocks;
    // Lane j holds the block-table entry of this warp's j-th tile (the first 32 tiles of a warp: 2048 positions), so
    // no table read sits between the end of one tile and the request for the next. Unsplit launches know which
    // entries those are without the length: they are fetched together with it (one memory latency instead of two
    // before the first tile can be requested). Entries past the sequence's end are never used.
    uint32_t my_blk = 0;
    if (n_splits == 1 && warp + lane * DEC_WARPS < max_blocks) my_blk = (uint32_t)table[warp + lane * DEC_WARPS];
    const int32_t kv_len = kv_lens[row];

    // block range of this split
    const uint32_t nblk = kv_len > 0 ? ((uint32_t)kv_len + DEC_BS - 1) / DEC_BS : 0;
    uint32_t n_act, bps;
    split_plan(nblk, n_splits, n_act, bps);
    if (split >= n_act) return;   // whole CTA: nothing to do for this (row, head)
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

    // blocks of this warp: b_begin + warp, + DEC_WARPS, ...
    const uint32_t first = b_begin + warp;
    const uint32_t nmine = (first < b_end) ? (b_end - first + DEC_WARPS - 1) / DEC_WARPS : 0;

    auto issue = [&](uint32_t i, uint32_t blk) {  // one lane
        const uint32_t s = i % C::STAGES;
        const int32_t y = (int32_t)((blk * heads + h) * DEC_BS);
        uint8_t* kdst = my_smem + (size_t)s * C::STAGE_BYTES;
        uint8_t* vdst = kdst + C::TILE_BYTES;
        mbar_expect_tx(&full_bar[warp][s], C::STAGE_BYTES);
#pragma unroll
        for (int g = 0; g < C::GROUPS; g++) {
            tma_load_2d(kdst + g * (DEC_BS * 128), &tmK, g * C::EPG, y, &full_bar[warp][s]);
            tma_load_2d(vdst + g * (DEC_BS * 128), &tmV, g * C::EPG, y, &full_bar[warp][s]);
        }
    };

    // first ring of loads, one lane per stage (each reads its own block-table entry); the block that
    // holds the newest position (written by the preceding kernel) is held back until that kernel is
    // known to be complete
    const uint32_t pre = nmine < (uint32_t)C::STAGES ? nmine : (uint32_t)C::STAGES;
    bool deferred = false;
    if (n_splits != 1 && lane < nmine) my_blk = (uint32_t)table[first + lane * DEC_WARPS];
    // physical block of this warp's j-th tile (j warp-uniform)
    auto blk_of = [&](uint32_t j) { return j < 32 ? __shfl_sync(0xffffffffu, my_blk, j) : (uint32_t)table[first + j * DEC_WARPS]; };
    if (lane < pre) {
        deferred = early && !fused && (first + lane * DEC_WARPS + 1 == nblk);
        if (!deferred) issue(lane, my_blk);
    }
    if (early) pdl_wait();
    if (deferred) issue(lane, my_blk);
    __syncwarp();

    float m_run = -INFINITY, l_run = 0.0f;
    bool failed = false;
    const T* qrow = q + ((size_t)row * heads + h) * HD;
    // fused form: this head's slices of the new token's q | k | v, and the RoPE factors of its position
    const uint32_t dim = heads * HD;
    const float* q32 = fused ? fz.qkv + (size_t)row * 3 * dim + (size_t)h * HD : nullptr;
    const uint32_t new_pos = kv_len > 0 ? (uint32_t)kv_len - 1 : 0;
    const float2* cs_row = fused ? fz.rope + (size_t)(new_pos < fz.rope_len ? new_pos : 0) * (HD / 2) : nullptr;
    // q elements d, d+1 (d even) after RoPE, in the fused form
    auto q_pair = [&](uint32_t d, float& a, float& b) {
        const float2 x = *reinterpret_cast<const float2*>(q32 + d);
        const float2 f = cs_row[d >> 1];
        rope_rotate(x.x, x.y, f.x, f.y, a, b);
    };
    // The warp that owns the block holding the new position: rotate the new key, store the new key and value rows to
    // the pools and patch them into the tile in shared memory (the tile was requested before they existed).
    auto append_new = [&](uint32_t blk_phys, uint8_t* k_tile, uint8_t* v_tile) {
        constexpr uint32_t CH = HD * (uint32_t)sizeof(T) / 16;   // 16-byte chunks per row
        const uint32_t within = new_pos & (DEC_BS - 1);
        for (uint32_t c = lane; c < 2 * CH; c += 32) {
            const bool is_v = c >= CH;
            const uint32_t cc = is_v ? c - CH : c, d0 = cc * C::EPC;
            const float* src = q32 + (is_v ? 2 : 1) * dim + d0;
            float x[C::EPC];
#pragma unroll
            for (int e = 0; e < C::EPC; e += 4) {
                const float4 t4 = *reinterpret_cast<const float4*>(src + e);
                x[e] = t4.x; x[e + 1] = t4.y; x[e + 2] = t4.z; x[e + 3] = t4.w;
            }
            if (!is_v) {
#pragma unroll
                for (int e = 0; e < C::EPC; e += 2) {
                    const float2 f = cs_row[(d0 + e) >> 1];
                    rope_rotate(x[e], x[e + 1], f.x, f.y, x[e], x[e + 1]);
                }
            }
            alignas(16) T o[C::EPC];
#pragma unroll
            for (int e = 0; e < C::EPC; e++) o[e] = Cvt<T>::from_f(x[e]);
            const uint4 pk = *reinterpret_cast<const uint4*>(o);
            T* pool = reinterpret_cast<T*>(is_v ? fz.v_pool : fz.k_pool);
            *reinterpret_cast<uint4*>(pool + (((size_t)blk_phys * heads + h) * DEC_BS + within) * HD + d0) = pk;
            uint8_t* tile = is_v ? v_tile : k_tile;
            *reinterpret_cast<uint4*>(tile + (cc >> 3) * (DEC_BS * 128) + within * 128 + (((cc & 7) ^ (within & 7)) << 4)) = pk;
        }
        __syncwarp();
    };

    if constexpr (MMA) {
        // ---------------- bf16: tensor-core tiles -------------------------------------------------
        constexpr int KS = HD / 16;   // k-steps of Q.K^T
        constexpr int NT = HD / 8;    // 8-wide output tiles of P.V
        const uint32_t g8 = lane >> 2, t4 = lane & 3;
        (void)g8;
        // A operand of Q.K^T: every row is q, so a0 == a1 and a2 == a3
        uint32_t qa[KS][2];
        if (fused) {
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                float a, b;
                q_pair(ks * 16 + 2 * t4, a, b);
                qa[ks][0] = pack_bf16x2(a, b);
                q_pair(ks * 16 + 8 + 2 * t4, a, b);
                qa[ks][1] = pack_bf16x2(a, b);
            }
        } else {
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                qa[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
                qa[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t4);
            }
        }
        // per-lane ldmatrix row addresses inside a tile (swizzled): matrix mi = lane / 8, row r = lane % 8
        const uint32_t mi = lane >> 3, r8 = lane & 7;
        // K (no transpose): matrices (pos 0-7, lo dims), (pos 0-7, hi dims), (pos 8-15, lo), (pos 8-15, hi)
        const uint32_t k_pos = r8 + 8 * (mi >> 1), k_csel = mi & 1;
        // V (transpose): matrices (pos 0-7, chunk c), (pos 8-15, chunk c), (pos 0-7, chunk c+1), (pos 8-15, chunk c+1)
        const uint32_t v_pos = r8 + 8 * (mi & 1), v_csel = mi >> 1;
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f; }
        const float sl2 = scale * 1.4426950408889634f;   // scores in the base-2 domain

        for (uint32_t i = 0; i < nmine; i++) {
            const uint32_t s = i % C::STAGES;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[warp][s], (i / C::STAGES) & 1u));
            if (!ok) { failed = true; break; }
            const uint32_t ksm = smem_u32(my_smem + (size_t)s * C::STAGE_BYTES);
            const uint32_t vsm = ksm + C::TILE_BYTES;
            const uint32_t blk_idx = first + i * DEC_WARPS;
            const int32_t n_valid_raw = kv_len - (int32_t)(blk_idx * DEC_BS);
            const uint32_t n_valid = n_valid_raw >= DEC_BS ? DEC_BS : (uint32_t)n_valid_raw;
            if (fused && blk_idx + 1 == nblk)
                append_new(blk_of(i), my_smem + (size_t)s * C::STAGE_BYTES, my_smem + (size_t)s * C::STAGE_BYTES + C::TILE_BYTES);
            if (n_valid < DEC_BS) {
                // rows past the end of the sequence may hold anything (their probability is 0, but
                // 0 * NaN would poison the tensor-core sum): clear them in the V tile
                uint8_t* vgen = my_smem + (size_t)s * C::STAGE_BYTES + C::TILE_BYTES;
                for (uint32_t c = lane; c < (DEC_BS - n_valid) * 8 * C::GROUPS; c += 32) {
                    const uint32_t rr = n_valid + c / (8 * C::GROUPS), rem = c % (8 * C::GROUPS);
                    *reinterpret_cast<uint4*>(vgen + (rem >> 3) * (DEC_BS * 128) + rr * 128 + (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            // ---- S = q . K^T : sc[0] = positions 0-7, sc[1] = positions 8-15; this lane's columns 2*t4, 2*t4+1
            float sc[2][4];
            sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = 0.0f;
            sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                const uint32_t grp = (2 * ks) >> 3, chunk = ((2 * ks) & 7) + k_csel;
                uint32_t kb[4];
                ldsm_x4(ksm + grp * (DEC_BS * 128) + k_pos * 128 + ((chunk ^ (k_pos & 7)) << 4), kb);
                mma_bf16_16816(sc[0], qa[ks][0], qa[ks][0], qa[ks][1], qa[ks][1], kb[0], kb[1]);
                mma_bf16_16816(sc[1], qa[ks][0], qa[ks][0], qa[ks][1], qa[ks][1], kb[2], kb[3]);
            }
            float s0 = sc[0][0] * sl2, s1 = sc[0][1] * sl2, s2 = sc[1][0] * sl2, s3 = sc[1][1] * sl2;
            if (n_valid < DEC_BS) {
                if (2 * t4 >= n_valid) s0 = -INFINITY;
                if (2 * t4 + 1 >= n_valid) s1 = -INFINITY;
                if (8 + 2 * t4 >= n_valid) s2 = -INFINITY;
                if (9 + 2 * t4 >= n_valid) s3 = -INFINITY;
            }
            // ---- online softmax (the 4 lanes of a quad hold the 16 positions; quads are replicas)
            float mb = fmaxf(fmaxf(s0, s1), fmaxf(s2, s3));
            mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
            mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
            const float m_new = fmaxf(m_run, mb);
            const float corr = fast_ex2(m_run - m_new);   // ex2(-inf) = 0 on the first block
            const uint32_t p01 = pack_bf16x2(fast_ex2(s0 - m_new), fast_ex2(s1 - m_new));
            const uint32_t p23 = pack_bf16x2(fast_ex2(s2 - m_new), fast_ex2(s3 - m_new));
            // the row sum adds the bf16-rounded probabilities, the values the tensor core multiplies
            float lb = __uint_as_float(p01 << 16) + __uint_as_float(p01 & 0xffff0000u) + __uint_as_float(p23 << 16) +
                       __uint_as_float(p23 & 0xffff0000u);
            lb += __shfl_xor_sync(0xffffffffu, lb, 1);
            lb += __shfl_xor_sync(0xffffffffu, lb, 2);
            l_run = l_run * corr + lb;
            if (m_new != m_run) {   // warp-uniform
#pragma unroll
                for (int j = 0; j < NT; j++) { acc[j][0] *= corr; acc[j][1] *= corr; }
            }
            m_run = m_new;
            // ---- O += P . V
#pragma unroll
            for (int jj = 0; jj < NT / 2; jj++) {
                const uint32_t grp = (2 * jj) >> 3, chunk = ((2 * jj) & 7) + v_csel;
                uint32_t vb[4];
                ldsm_x4_trans(vsm + grp * (DEC_BS * 128) + v_pos * 128 + ((chunk ^ (v_pos & 7)) << 4), vb);
                mma_bf16_16816(acc[2 * jj], p01, p01, p23, p23, vb[0], vb[1]);
                mma_bf16_16816(acc[2 * jj + 1], p01, p01, p23, p23, vb[2], vb[3]);
            }
            __syncwarp();
            if (i + C::STAGES < nmine) {   // warp-uniform
                const uint32_t nb = blk_of(i + C::STAGES);
                if (lane == 0) issue(i + C::STAGES, nb);
            }
        }
        // rows of the accumulator are replicas: quad 0 (lanes 0-3) publishes the warp's output
        if (lane < 4) {
#pragma unroll
            for (int j = 0; j < NT; j++) {
                sm_acc[warp][8 * j + 2 * lane] = acc[j][0];
                sm_acc[warp][8 * j + 2 * lane + 1] = acc[j][1];
            }
        }
    } else {
        // ---------------- f32 (parity mode): scalar FMAs, 2 lanes per position ---------------------
        const uint32_t p = lane >> 1, hh = lane & 1;
        float qreg[C::QREGS];
#pragma unroll
        for (int g = 0; g < C::GROUPS; g++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                if (fused) {
                    // the rotated value is rounded to the cache dtype, as the unfused path stores and re-reads it
#pragma unroll
                    for (int e = 0; e < C::EPC; e += 2) {
                        float a, b;
                        q_pair(g * C::EPG + (4 * hh + c) * C::EPC + e, a, b);
                        qreg[(g * 4 + c) * C::EPC + e] = Cvt<T>::to_f(Cvt<T>::from_f(a));
                        qreg[(g * 4 + c) * C::EPC + e + 1] = Cvt<T>::to_f(Cvt<T>::from_f(b));
                    }
                } else {
                    uint4 raw = *reinterpret_cast<const uint4*>(qrow + g * C::EPG + (4 * hh + c) * C::EPC);
                    unpack16<T>(raw, &qreg[(g * 4 + c) * C::EPC]);
                }
            }
        float acc[C::EPL];
#pragma unroll
        for (int e = 0; e < C::EPL; e++) acc[e] = 0.0f;

        for (uint32_t i = 0; i < nmine; i++) {
            const uint32_t s = i % C::STAGES;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[warp][s], (i / C::STAGES) & 1u));
            if (!ok) { failed = true; break; }
            const uint8_t* ksm = my_smem + (size_t)s * C::STAGE_BYTES;
            const uint8_t* vsm = ksm + C::TILE_BYTES;
            const uint32_t blk_idx = first + i * DEC_WARPS;
            const int32_t n_valid_raw = kv_len - (int32_t)(blk_idx * DEC_BS);
            const uint32_t n_valid = n_valid_raw >= DEC_BS ? DEC_BS : (uint32_t)n_valid_raw;
            if (fused && blk_idx + 1 == nblk)
                append_new(blk_of(i), my_smem + (size_t)s * C::STAGE_BYTES, my_smem + (size_t)s * C::STAGE_BYTES + C::TILE_BYTES);

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
                constexpr int LB = C::EPL * (int)sizeof(T);  // bytes per lane per row (8 or 16)
                const uint32_t byte_off = lane * LB;
                const uint32_t g = byte_off >> 7, cin = (byte_off & 127) >> 4, within = byte_off & 15;
                const uint8_t* vbase = vsm + g * (DEC_BS * 128) + within;
#pragma unroll
                for (int j = 0; j < DEC_BS; j++) {
                    const float pw = __shfl_sync(0xffffffffu, pj, 2 * j);
                    if ((uint32_t)j < n_valid) {
                        const uint8_t* vp = vbase + j * 128 + ((cin ^ (j & 7)) << 4);
                        if constexpr (LB == 8) {
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
            if (i + C::STAGES < nmine) {   // warp-uniform
                const uint32_t nb = blk_of(i + C::STAGES);
                if (lane == 0) issue(i + C::STAGES, nb);
            }
        }
#pragma unroll
        for (int e = 0; e < C::EPL; e++) sm_acc[warp][lane * C::EPL + e] = acc[e];
    }
    if (failed) {   // warp-uniform
        if (lane == 0) atomicExch(&g_attn_decode_status, 1u);
        // give the copies still in flight one more bounded chance to land before leaving
        for (uint32_t i2 = 0; i2 < (uint32_t)C::STAGES; i2++) (void)mbar_wait(&full_bar[warp][i2], 0);
        __syncwarp();
    }

    // ---- merge the four warps
    if (lane == 0) { sm_m[warp] = m_run; sm_l[warp] = l_run; }
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
        finish_row<T, HD>(M, L, o, out, scratch, row, h, heads, gridDim.y, split, n_splits, n_act, lane);
    }
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
    return partial_floats(rows, heads, head_dim, n_splits) * sizeof(float) + (size_t)rows * heads * sizeof(unsigned int);
}

// Launch plan. The kernel's time is set by how many WAVES of CTAs the launch needs and by the longest chain of
// ring rounds inside one CTA, not by bytes alone: a CTA's life is a chain of memory latencies (lengths and block
// table, first tiles, one ring round per 2 blocks of a warp, merge). So: a 2-deep ring per warp (33 KB per CTA with
// bf16 head_dim 64: 6 CTAs = 24 warps per SM, 888 slots, a 64-sequence x 12-head batch is ONE wave), and sequences
// are split over several CTAs only while all CTAs still fit one wave (a single sequence or a handful of them: one CTA
// per (sequence, head) would leave most SMs idle and run the whole length serially).
constexpr uint32_t DEC_STAGES = 2;   // measured: a 4-deep ring (3 CTAs per SM) needs two waves for the same batch and is slower
static uint32_t stage_bytes_of(uint32_t head_dim, uint32_t kv_dtype) { return 2 * DEC_BS * head_dim * (kv_dtype == AK_F32 ? 4 : 2); }
static uint32_t wave_slots(uint32_t head_dim, uint32_t kv_dtype, uint32_t stages) {
    const uint32_t smem = DEC_WARPS * stages * stage_bytes_of(head_dim, kv_dtype) + 1024 + 2048;
    uint32_t per_sm = (227 * 1024) / smem;
    if (per_sm > 6) per_sm = 6;
    if (per_sm < 1) per_sm = 1;
    return B200_SMS * per_sm;
}
uint32_t attn_decode_pick_splits(uint32_t rows, uint32_t heads, uint32_t head_dim, uint32_t kv_dtype, uint32_t max_kv_len) {
    const uint64_t items = (uint64_t)rows * heads;
    if (items == 0) return 1;
    const uint32_t st = DEC_STAGES;
    const uint32_t room = (uint32_t)(wave_slots(head_dim, kv_dtype, st) / items);   // CTAs per item that keep one wave
    const uint32_t max_blocks = (max_kv_len + DEC_BS - 1) / DEC_BS;
    uint32_t want = (max_blocks + DEC_WARPS * st - 1) / (DEC_WARPS * st);           // every warp at most one ring of blocks
    if (want > room) want = room;
    if (want > DEC_MAX_SPLITS) want = DEC_MAX_SPLITS;
    return want < 1 ? 1 : want;
}

template <typename T, int HD, int ST>
static int launch_fast_st(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                          const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                          const ak_attn_decode_params& p, uint32_t n_splits, uint64_t pool_rows, const DecFused& fz) {
    using C = DecCfg<T, HD, ST>;
    CUtensorMap tmK, tmV;
    int rc = make_tmap_2d(&tmK, k_pool, sizeof(T), HD, pool_rows, (uint64_t)HD * sizeof(T), C::EPG, DEC_BS, TMA_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&tmV, v_pool, sizeof(T), HD, pool_rows, (uint64_t)HD * sizeof(T), C::EPG, DEC_BS, TMA_SWIZZLE_128B);
    if (rc) return rc;
    {
        static bool attr_set[64] = {};
        int dev = 0;
        AK_CUDA(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(device_cache_mutex());
        if (!attr_set[dev & 63]) {
            AK_CUDA(cudaFuncSetAttribute(attn_decode_paged_kernel<T, HD, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
            attr_set[dev & 63] = true;
        }
    }
    dim3 grid(p.heads, p.rows, n_splits);
    return launch_k(attn_decode_paged_kernel<T, HD, ST>, dim3(grid), dim3(DEC_WARPS * 32), C::SMEM_BYTES, st, NO_CLUSTER, tmK, tmV,
                    (const T*)q, block_tables, kv_lens, (T*)out, (float*)scratch, p.heads, p.max_blocks_per_seq, p.scale, n_splits,
                    (uint32_t)(g_attn_early ? 1 : 0), fz);
}

template <typename T, int HD>
static int launch_fast(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                       const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                       const ak_attn_decode_params& p, uint32_t n_splits, uint64_t pool_rows, const DecFused& fz) {
    return launch_fast_st<T, HD, (int)DEC_STAGES>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, pool_rows, fz);
}

// Rows of the 2-D view [n_blocks*heads*16, head_dim] of a pool. With pool_blocks given, a block
// id outside the pool reads zeros (TMA out-of-range fill) instead of touching foreign memory.
static uint64_t pool_rows_bound(const ak_attn_decode_params& p) {
    if (p.pool_blocks) return (uint64_t)p.pool_blocks * p.heads * DEC_BS;
    return (uint64_t)1 << 31;
}

static int launch_decode(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                         const ak_attn_decode_params& p, bool counters_are_zero, const DecFused& fz);

bool attn_decode_fused_supported(uint32_t head_dim) { return head_dim == 64 || head_dim == 128; }

// CTAs are handed to the SMs in launch order, one per SM and round: CTA number c = y * heads + h lands on SM c mod 148
// as that SM's (c / 148)-th CTA. A launch that fits one wave therefore gives every SM one row out of each "level" of
// 148 / heads consecutive y. Rows sorted by length are dealt to the levels in a snake (level 0 longest first, level 1
// shortest first, ...), so every SM gets a long row with a short one and the last, partly filled level holds the
// shortest rows. A launch of several waves gets the longest rows first (the short ones fill the tail).
void attn_decode_row_order(const int32_t* kv_lens, uint32_t rows, uint32_t heads, uint32_t head_dim, uint32_t kv_dtype, int32_t* order_out) {
    std::vector<uint32_t> by_len(rows);
    for (uint32_t i = 0; i < rows; i++) by_len[i] = i;
    std::stable_sort(by_len.begin(), by_len.end(), [&](uint32_t a, uint32_t b) { return kv_lens[a] > kv_lens[b]; });
    const bool one_wave = (uint64_t)rows * heads <= wave_slots(head_dim, kv_dtype, DEC_STAGES);
    if (!one_wave || heads == 0) {
        for (uint32_t i = 0; i < rows; i++) order_out[i] = (int32_t)by_len[i];
        return;
    }
    // positions y in the order in which the sorted rows are dealt: by level, alternating direction
    std::vector<uint32_t> pos(rows);
    for (uint32_t y = 0; y < rows; y++) pos[y] = y;
    auto level = [&](uint32_t y) { return (uint32_t)(((uint64_t)y * heads) / B200_SMS); };
    std::stable_sort(pos.begin(), pos.end(), [&](uint32_t a, uint32_t b) {
        const uint32_t la = level(a), lb = level(b);
        if (la != lb) return la < lb;
        return (la & 1u) ? a > b : a < b;
    });
    for (uint32_t i = 0; i < rows; i++) order_out[pos[i]] = (int32_t)by_len[i];
}

int launch_attn_decode_paged(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                             const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                             const ak_attn_decode_params& p, bool counters_are_zero) {
    return launch_decode(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, counters_are_zero, DecFused{});
}

int launch_attn_decode_fused(cudaStream_t st, const float* qkv, const float2* rope_table, uint32_t rope_len, void* k_pool, void* v_pool,
                             const int32_t* block_tables, const int32_t* kv_lens, const int32_t* row_order, void* out, void* scratch,
                             const ak_attn_decode_params& p, bool counters_are_zero) {
    AK_REQUIRE(attn_decode_fused_supported(p.head_dim) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) && ((uintptr_t)qkv % 16 == 0),
               AK_ERR_UNSUPPORTED, "attn_decode_fused: head_dim must be 64 or 128 and the buffers 16-byte aligned");
    AK_REQUIRE(rope_table && rope_len, AK_ERR_INVALID_ARG, "attn_decode_fused: a RoPE table is required");
    DecFused fz{row_order, qkv, rope_table, rope_len, k_pool, v_pool};
    return launch_decode(st, qkv, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, counters_are_zero, fz);
}

static int launch_decode(cudaStream_t st, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch,
                         const ak_attn_decode_params& p, bool counters_are_zero, const DecFused& fz) {
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
    const uint32_t n_splits = p.n_splits ? p.n_splits : attn_decode_pick_splits(p.rows, p.heads, p.head_dim, p.kv_dtype, p.max_blocks_per_seq * DEC_BS);
    AK_REQUIRE(n_splits <= DEC_MAX_SPLITS, AK_ERR_INVALID_ARG, "attn_decode_paged: n_splits must be at most %d", DEC_MAX_SPLITS);
    AK_REQUIRE(n_splits == 1 || scratch, AK_ERR_INVALID_ARG, "attn_decode_paged: scratch required when n_splits > 1");
    if (n_splits > 1 && !counters_are_zero) {
        // the arrival counters behind the partials must start at zero (the kernel leaves them at zero)
        AK_CUDA(cudaMemsetAsync((float*)scratch + partial_floats(p.rows, p.heads, p.head_dim, n_splits), 0,
                                (size_t)p.rows * p.heads * sizeof(unsigned int), st));
    }
    const uint64_t rows_bound = pool_rows_bound(p);
    if (p.kv_dtype == AK_F32) {
        if (p.head_dim == 64) return launch_fast<float, 64>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, rows_bound, fz);
        return launch_fast<float, 128>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, rows_bound, fz);
    }
    if (p.head_dim == 64) return launch_fast<bf16, 64>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, rows_bound, fz);
    return launch_fast<bf16, 128>(st, q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, n_splits, rows_bound, fz);
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
    uint32_t ns = p->n_splits ? p->n_splits : attn_decode_pick_splits(p->rows, p->heads, p->head_dim, p->kv_dtype, p->max_blocks_per_seq * DEC_BS);
    return attn_decode_scratch_bytes(p->rows, p->heads, p->head_dim, ns);
}
int ak_attn_decode_paged(void* stream, const void* q, const void* k_pool, const void* v_pool, const int32_t* block_tables,
                         const int32_t* kv_lens, void* out, void* scratch, ak_attn_decode_params p) {
    AK_REQUIRE(q && k_pool && v_pool && block_tables && kv_lens && out, AK_ERR_INVALID_ARG, "ak_attn_decode_paged: null pointer");
    return launch_attn_decode_paged(as_stream(stream), q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, false);
}
int ak_attn_decode_append_paged(void* stream, const float* qkv, const float* rope_table, uint32_t rope_len, void* k_pool, void* v_pool,
                                const int32_t* block_tables, const int32_t* kv_lens, void* out, void* scratch, ak_attn_decode_params p) {
    AK_REQUIRE(qkv && rope_table && k_pool && v_pool && block_tables && kv_lens && out, AK_ERR_INVALID_ARG, "ak_attn_decode_append_paged: null pointer");
    AK_REQUIRE(p.block_size == DEC_BS && p.kv_dtype <= AK_BF16, AK_ERR_INVALID_ARG, "ak_attn_decode_append_paged: block_size must be 16, kv_dtype f32 or bf16");
    return launch_attn_decode_fused(as_stream(stream), qkv, reinterpret_cast<const float2*>(rope_table), rope_len, k_pool, v_pool, block_tables,
                                    kv_lens, nullptr, out, scratch, p, false);
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
    std::lock_guard<std::mutex> lock(device_cache_mutex());
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
    const uint32_t ns = p.n_splits ? p.n_splits : attn_decode_pick_splits(p.rows, p.heads, p.head_dim, p.kv_dtype, p.max_blocks_per_seq * DEC_BS);
    const size_t need = attn_decode_scratch_bytes(p.rows, p.heads, p.head_dim, ns);
    AK_REQUIRE(need <= AK_NOALLOC_SCRATCH_BYTES, AK_ERR_UNSUPPORTED,
               "ak_attn_decode_paged_noalloc: %zu bytes of split partials and arrival counters exceed the built-in "
               "%zu-byte buffer; lower n_splits or use ak_attn_decode_paged with caller scratch",
               need, (size_t)AK_NOALLOC_SCRATCH_BYTES);
    void* scratch = nullptr;
    int rc = noalloc_scratch_ptr(&scratch);
    if (rc) return rc;
    p.n_splits = ns;
    // Every partial that is read was written earlier in the same call, so the previous call's partials never
    // matter. The arrival counters behind them must start at zero: the launch clears them on the stream first
    // (a memset, not an allocation), whatever an earlier, possibly failed, call left there.
    return launch_attn_decode_paged(as_stream(stream), q, k_pool, v_pool, block_tables, kv_lens, out, scratch, p, false);
}
}
