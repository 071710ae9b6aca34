// Causal varlen prefill attention on the 5th-generation tensor cores (bf16 K/V/Q, fp32 softmax):
// the same online-softmax recurrence as the reference's FLASH_ATTENTION kernel
// (src/shaders/cuda.rs:633-685), tiled 128 queries x BKV keys (BKV = 64 or 128).
//
// One CTA (4 warps, thread <-> query row <-> TMEM lane) per (128-query tile, head, sequence):
//   * TMA: the Q tile once; per step a BKV-key K tile and V tile straight from the paged pools
//     (BKV/16 blocks of 16 positions, 128-byte swizzle), double-buffered.
//   * S = Q.K^T  : tcgen05.mma, A = Q (K-major), B = K tile (K-major), fp32 in TMEM columns [0,BKV).
//   * softmax    : each thread reads ITS row of S with tcgen05.ld (no cross-thread reduction),
//                  applies scale + causal mask, updates running max / sum, writes P (bf16) into
//                  shared memory in the swizzled K-major layout the next MMA reads.
//   * PV = P.V   : tcgen05.mma, A = P, B = V tile used as an MN-major operand (V rows are keys, the
//                  contiguous direction is head_dim), fp32 in TMEM columns [BKV, BKV+head_dim).
//   * O = O*corr + PV in registers; final O / sum -> bf16.
// All mbarrier waits are bounded; on expiry a status word is set and the CTA unwinds.
#include "kernels.h"
#include "tma.h"

namespace ak {

__device__ unsigned int g_prefill_tc_status = 0;

namespace pftc {

constexpr int BQ = 128, BS = 16, THREADS = 128;

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ float ex2(float x) {   // 2^x, hardware approximation (2 ulp), ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major operand, 128-byte swizzle, 128-byte rows; 8-row atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand (the contiguous direction is N): rows of the tile are K (keys), 128-byte swizzle;
// atoms of 8 K-rows are 1024 bytes apart (stride offset), the next 64-column slab along N starts
// `lbo` bytes further (leading offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: D f32, A/B bf16, A K-major, B K-major (b_mn = 0) or MN-major (1).
__host__ __device__ constexpr uint32_t idesc(uint32_t m, uint32_t n, uint32_t b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// BKV = keys per step = N of the QK^T instruction. One tcgen05.mma costs about the same for N = 64 and
// N = 128, and every step pays fixed latencies (commit -> wait, two CTA barriers), so wider is better
// until shared memory runs out.
template <int HD, int BKV> struct Cfg {
    static constexpr int HALVES = HD / 64;                 // 64-column (128-byte) slabs per row
    static constexpr int Q_BYTES = BQ * HD * 2;            // HALVES slabs of [128 x 64]
    static constexpr int KV_BYTES = BKV * HD * 2;          // HALVES slabs of [BKV x 64]
    static constexpr int P_BYTES = BQ * BKV * 2;           // BKV/64 slabs of [128 x 64]
    static constexpr int SMEM_BYTES = Q_BYTES + 2 * 2 * KV_BYTES + P_BYTES + 1024;
    static constexpr int TMEM_COLS = (BKV + HD) <= 128 ? 128 : ((BKV + HD) <= 256 ? 256 : 512);
};

template <int HD, int BKV>
__global__ void __launch_bounds__(THREADS)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const int32_t* __restrict__ block_tables, uint32_t max_blocks,
                  const int32_t* __restrict__ cu, const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ q_pos0,
                  bf16* __restrict__ out, uint32_t row_base, uint32_t heads, float scale) {
    using C = Cfg<HD, BKV>;
    pdl_wait();
    extern __shared__ uint8_t smem_raw[];

    const uint32_t seq = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BQ;
    // len query rows at positions pos0 .. pos0 + len - 1 (pos0 > 0: a later chunk of a prompt whose first pos0
    // positions are already in the cache); keys are positions 0 .. kv_len - 1
    const uint32_t len = (uint32_t)(cu[seq + 1] - cu[seq]);
    const uint32_t pos0 = q_pos0 ? (uint32_t)q_pos0[seq] : 0u;
    const uint32_t kv_len = pos0 + len;
    if (q0 >= len) { pdl_trigger(); return; }   // allocates no TMEM
    const uint32_t row0 = row_base + (uint32_t)cu[seq];
    const int32_t* table = block_tables + (size_t)seq_slot[seq] * max_blocks;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t dim = heads * HD;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_sm = smem;
    uint8_t* kv_sm = q_sm + C::Q_BYTES;            // [buf][K | V] each KV_BYTES
    uint8_t* p_sm = kv_sm + 4 * C::KV_BYTES;
    // The barriers live in the dynamic allocation too, behind the tiles: with no static shared memory at all the
    // 112 KB of tiles + 1 KB of alignment room are exactly what lets TWO CTAs share an SM (228 KB, 1 KB reserved per
    // CTA); 48 bytes of static variables made it one. The room left for alignment is 1024 - 64 bytes, enough for any
    // base that is 64-byte aligned (with nothing static in front of it the base is the start of the CTA's window).
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_sm + C::P_BYTES);
    uint64_t& q_bar = bars[0];
    uint64_t* kv_bar = bars + 1;   // [2]
    uint64_t& s_bar = bars[3];
    uint64_t& pv_bar = bars[4];
    uint32_t& tmem_base_sm = *reinterpret_cast<uint32_t*>(bars + 5);
    uint32_t& fail_flag = *(reinterpret_cast<uint32_t*>(bars + 5) + 1);
    if ((uintptr_t)(smem - smem_raw) > 1024 - 64) {   // cannot happen with the alignment above; never run past the allocation
        if (tid == 0) atomicExch(&g_prefill_tc_status, 9u);
        pdl_trigger();
        return;
    }

    if (tid == 0) {
        mbar_init(&q_bar, 1); mbar_init(&kv_bar[0], 1); mbar_init(&kv_bar[1], 1); mbar_init(&s_bar, 1); mbar_init(&pv_bar, 1);
        fail_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) { tmem_alloc(&tmem_base_sm, C::TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Invariant of every TMEM-using kernel of this library: dependents are released only AFTER this CTA holds its
    // TMEM columns. A dependent grid's CTAs allocate TMEM and then block in griddepcontrol.wait until this grid
    // has completed; were they let in first, they could take the columns this CTA still needs and both would wait.
    pdl_trigger();
    const uint32_t tmem_s = tmem_base_sm, tmem_pv = tmem_base_sm + BKV;
    const uint32_t lane_addr = (warp * 32u) << 16;

    const uint32_t q_hi = pos0 + ((q0 + BQ - 1 < len - 1) ? q0 + BQ - 1 : len - 1);   // position of the tile's last query
    const uint32_t n_tiles = q_hi / BKV + 1;

    uint32_t loaded = 0, consumed = 0;  // warp 0: K/V tiles requested / waited for
    // Called by the whole of warp 0: lane 0 arms the barrier, then one lane per 16-position block looks up its block
    // and requests its K and V rows (a single thread issuing all 16 loads of a tile one after the other spent
    // ~1200 cycles on it, on the path of every tile).
    auto load_kv = [&](uint32_t t) {
        loaded = t + 1;
        const uint32_t b = t & 1, lane = tid & 31;
        uint8_t* k_dst = kv_sm + (size_t)b * 2 * C::KV_BYTES;
        uint8_t* v_dst = k_dst + C::KV_BYTES;
        if (lane == 0) mbar_expect_tx(&kv_bar[b], 2 * C::KV_BYTES);
        __syncwarp();
        if (lane < BKV / BS) {
            const uint32_t blk = lane;
            const uint32_t pos = t * BKV + blk * BS;
            // blocks past the sequence end are fetched from its first block: finite data, masked out below
            const uint32_t bidx = pos < kv_len ? pos / BS : 0;
            const int32_t y = (int32_t)(((uint32_t)table[bidx] * heads + h) * BS);
#pragma unroll
            for (int hf = 0; hf < C::HALVES; hf++) {
                tma_load_2d(k_dst + hf * (BKV * 128) + blk * (BS * 128), &tmK, hf * 64, y, &kv_bar[b]);
                tma_load_2d(v_dst + hf * (BKV * 128) + blk * (BS * 128), &tmV, hf * 64, y, &kv_bar[b]);
            }
        }
    };

    if (warp == 0) {
        if (tid == 0) {
            mbar_expect_tx(&q_bar, C::Q_BYTES);
#pragma unroll
            for (int hf = 0; hf < C::HALVES; hf++)
                tma_load_2d(q_sm + hf * (BQ * 128), &tmQ, (int32_t)(h * HD + hf * 64), (int32_t)(row0 + q0), &q_bar);
        }
        load_kv(0);
    }

    float o[HD];
#pragma unroll
    for (int d = 0; d < HD; d++) o[d] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;   // m_run in the base-2 domain (score * scale * log2 e)
    const float sl2 = scale * 1.4426950408889634f;
    const uint32_t qi = pos0 + q0 + tid;  // this thread's query position
    bool ok = true;

    for (uint32_t t = 0; t < n_tiles; t++) {
        const uint32_t b = t & 1, ph = t & 1;
        uint8_t* k_sm = kv_sm + (size_t)b * 2 * C::KV_BYTES;
        uint8_t* v_sm = k_sm + C::KV_BYTES;
        if (warp == 0) {
          if (tid == 0) {
            bool w = (t > 0) || mbar_wait(&q_bar, 0);
            w = w && mbar_wait(&kv_bar[b], (t >> 1) & 1u);
            if (!w) atomicExch(&fail_flag, 1u);
            tc_fence_after();
            // S[128 x 64] = Q[128 x HD] . K[64 x HD]^T
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) {
                const uint32_t hf = kk / 4, ko = (kk % 4) * 2;
                tc_mma(tmem_s, desc_kmajor(smem_u32(q_sm + hf * (BQ * 128))) + ko, desc_kmajor(smem_u32(k_sm + hf * (BKV * 128))) + ko,
                       idesc(BQ, BKV, 0), kk != 0);
            }
            tc_commit(&s_bar);
          }
          // the next tile's K/V, requested while the tensor core works on S (the other buffer was released by pv_bar of
          // tile t-1, which every thread has waited for)
          __syncwarp();
          consumed = t + 1;
          if (t + 1 < n_tiles) load_kv(t + 1);
        }
        bool good = mbar_wait(&s_bar, ph);
        if (!good) atomicExch(&fail_flag, 2u);
        tc_fence_after();
        const uint32_t k0 = t * BKV;
        if (k0 + BKV > kv_len) {
            // Tile rows past the sequence end hold whatever the pool held (possibly non-finite): their
            // probabilities are 0, but 0 * NaN would poison P.V, so clear those V rows (whole 128-byte rows,
            // the swizzle permutes within a row only). Ordered before the MMA by the fence + barrier below.
            good = mbar_wait(&kv_bar[b], (t >> 1) & 1u) && good;
            const uint32_t first = kv_len - k0, chunks = (BKV - first) * 8;
            for (int hf = 0; hf < C::HALVES; hf++)
                for (uint32_t i = tid; i < chunks; i += THREADS)
                    *reinterpret_cast<uint4*>(v_sm + hf * (BKV * 128) + (first + i / 8) * 128 + (i % 8) * 16) = make_uint4(0, 0, 0, 0);
        }
        // A tile needs the per-element mask only if it reaches past the sequence end or past the first query of this
        // CTA's tile (the diagonal); every other tile is fully visible to every row. CTA-uniform.
        const bool need_mask = (k0 + BKV > kv_len) || (k0 + BKV - 1 > pos0 + q0);
        // ---- pass 1: row maximum of the raw scores (scale > 0: scaling commutes with the maximum)
        float mx = -INFINITY;
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < BKV; c0 += 32) {
            uint32_t r[32];
            tmem_ld16(tmem_s + lane_addr + c0, r);
            tmem_ld16(tmem_s + lane_addr + c0 + 16, r + 16);
            tmem_ld_wait();
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const uint32_t kj = k0 + c0 + j;
                    if (kj <= qi && kj < kv_len) mx = fmaxf(mx, __uint_as_float(r[j]));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) mx = fmaxf(mx, __uint_as_float(r[j]));
            }
        }
        // running maximum and exponentials in base 2: p = 2^(s * scale * log2(e) - m), one FMA and one ex2 per score
        const float m_new = fmaxf(m_run, mx * sl2);
        const float corr = (m_new == -INFINITY) ? 1.0f : ex2(m_run - m_new);
        // ---- pass 2: P = 2^(s * sl2 - m_new) -> bf16 -> shared (swizzled K-major rows of 128 bytes)
        float rs = 0.0f;
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < BKV; c0 += 32) {
            uint32_t r[32];
            tmem_ld16(tmem_s + lane_addr + c0, r);
            tmem_ld16(tmem_s + lane_addr + c0 + 16, r + 16);
            tmem_ld_wait();
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                float p2[2];
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float pe = ex2(fmaf(__uint_as_float(r[j + e]), sl2, -m_new));
                    const uint32_t kj = k0 + c0 + j + e;
                    p2[e] = (!need_mask || (kj <= qi && kj < kv_len)) ? pe : 0.0f;
                }
                bf162 v2 = __floats2bfloat162_rn(p2[0], p2[1]);
                // the running sum uses the ROUNDED probabilities, the ones the tensor core multiplies
                rs += __bfloat162float(v2.x) + __bfloat162float(v2.y);
                pk[j / 2] = *reinterpret_cast<uint32_t*>(&v2);
            }
            uint8_t* p_row = p_sm + (c0 / 64) * (BQ * 128) + tid * 128;  // slab of 64 keys, this thread's row
            const uint32_t ch = (c0 % 64) / 8;                           // four 16-byte chunks per 32 columns
#pragma unroll
            for (uint32_t q4 = 0; q4 < 4; q4++)
                *reinterpret_cast<uint4*>(p_row + (((ch + q4) ^ (tid & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        }
        l_run = l_run * corr + rs;
        m_run = m_new;
        fence_async_smem();  // generic-proxy writes of P must be visible to the tensor core (async proxy)
        tc_fence_before();
        if (__syncthreads_or(!good)) { ok = false; break; }  // every thread leaves together
        if (tid == 0) {
            tc_fence_after();
            // PV[128 x HD] = P[128 x 64] . V[64 x HD]   (V is the MN-major B operand)
#pragma unroll
            for (int kk = 0; kk < BKV / 16; kk++)
                tc_mma(tmem_pv, desc_kmajor(smem_u32(p_sm + (kk / 4) * (BQ * 128))) + (kk % 4) * 2, desc_mnmajor(smem_u32(v_sm + kk * (16 * 128)), BKV * 128),
                       idesc(BQ, HD, 1), kk != 0);
            tc_commit(&pv_bar);
        }
        good = mbar_wait(&pv_bar, ph);
        if (!good) atomicExch(&fail_flag, 3u);
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(tmem_pv + lane_addr + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j++) o[c0 + j] = fmaf(o[c0 + j], corr, __uint_as_float(r[j]));
        }
        tc_fence_before();
        // S and PV columns are free for the next tile, and so is the P buffer
        if (__syncthreads_or(!good)) { ok = false; break; }
    }

    if (!ok && tid == 0)  // leaving early: let the copies already requested land before the CTA's memory goes away
        for (uint32_t i = consumed; i < loaded; i++) mbar_wait(&kv_bar[i & 1], (i >> 1) & 1u);
    if (ok && q0 + tid < len) {
        const float inv = 1.0f / l_run;
        bf16* dst = out + (size_t)(row0 + q0 + tid) * dim + (size_t)h * HD;
#pragma unroll
        for (int d = 0; d < HD; d += 8) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                bf162 v2 = __floats2bfloat162_rn(o[d + 2 * e] * inv, o[d + 2 * e + 1] * inv);
                pk[e] = *reinterpret_cast<uint32_t*>(&v2);
            }
            *reinterpret_cast<uint4*>(dst + d) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && fail_flag) atomicExch(&g_prefill_tc_status, fail_flag);
    if (warp == 0) {
        __syncwarp();
        tmem_dealloc(tmem_base_sm, C::TMEM_COLS);
    }
}

template <int HD, int BKV>
static int launch(cudaStream_t st, const void* q, uint64_t q_rows, const void* k_pool, const void* v_pool, uint64_t pool_rows,
                  const int32_t* bt, uint32_t max_blocks, const int32_t* cu, const int32_t* seq_slot, const int32_t* pos0, void* out, uint32_t n_seqs,
                  uint32_t max_len, uint32_t row_base, uint32_t heads, float scale) {
    using C = Cfg<HD, BKV>;
    CUtensorMap tmQ, tmK, tmV;
    const uint64_t dim = (uint64_t)heads * HD;
    AK_TRY(make_tmap_2d(&tmQ, q, 2, dim, q_rows, dim * 2, 64, BQ, TMA_SWIZZLE_128B));
    AK_TRY(make_tmap_2d(&tmK, k_pool, 2, HD, pool_rows, (uint64_t)HD * 2, 64, BS, TMA_SWIZZLE_128B));
    AK_TRY(make_tmap_2d(&tmV, v_pool, 2, HD, pool_rows, (uint64_t)HD * 2, 64, BS, TMA_SWIZZLE_128B));
    static bool attr_set[64] = {};
    int dev = 0;
    AK_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(device_cache_mutex());
    if (!attr_set[dev & 63]) {
        AK_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<HD, BKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        attr_set[dev & 63] = true;
    }
    return launch_k(prefill_tc_kernel<HD, BKV>, dim3(cdiv(max_len, BQ), heads, n_seqs), dim3(THREADS), C::SMEM_BYTES, st, NO_CLUSTER, tmQ, tmK,
                    tmV, bt, max_blocks, cu, seq_slot, pos0, (bf16*)out, row_base, heads, scale);
}

}  // namespace pftc

int launch_attn_prefill_tc(cudaStream_t st, const void* q, uint64_t q_rows, const void* k_pool, const void* v_pool,
                           uint64_t pool_blocks, const int32_t* block_tables, uint32_t max_blocks_per_seq, const int32_t* cu,
                           const int32_t* seq_slot, const int32_t* pos0, void* out, uint32_t n_seqs, uint32_t max_len, uint32_t row_base, uint32_t heads,
                           uint32_t head_dim, float scale) {
    if (n_seqs == 0 || max_len == 0) return AK_OK;
    const uint64_t pool_rows = pool_blocks * heads * pftc::BS;
    // keys per step: 128 for head_dim 64 (a little faster); 64 for head_dim 128, where 128 would leave room for
    // one CTA per SM only (measured slower on long prompts).
#define AK_PF_ARGS st, q, q_rows, k_pool, v_pool, pool_rows, block_tables, max_blocks_per_seq, cu, seq_slot, pos0, out, n_seqs, max_len, row_base, heads, scale
    if (head_dim == 64) return pftc::launch<64, 128>(AK_PF_ARGS);
    AK_REQUIRE(head_dim == 128, AK_ERR_UNSUPPORTED, "prefill attention (tensor cores): head_dim must be 64 or 128");
    return pftc::launch<128, 64>(AK_PF_ARGS);
#undef AK_PF_ARGS
}

int prefill_tc_status(unsigned int* out) {
    AK_CUDA(cudaMemcpyFromSymbol(out, g_prefill_tc_status, sizeof(unsigned int)));
    return AK_OK;
}

}  // namespace ak
