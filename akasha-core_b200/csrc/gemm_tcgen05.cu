// bf16 tensor-core GEMM for sm_100a:  C[m,n] (op)= A[m,k] @ Wt[n,k]^T, fp32 accumulate.
//
// Both operands are K-major (row-major [rows, k]); tiles are staged into shared memory by TMA
// with the 128-byte swizzle, multiplied with tcgen05.mma (cta_group::1, kind::f16, M = 128)
// into a TMEM accumulator, and read back with tcgen05.ld for the fused epilogue
// (store f32 / += f32 residual / store bf16 / SiLU -> bf16).
//
// CTA = 6 warps: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM alloc/free),
// warps 2..5 = epilogue (each owns the TMEM lane quadrant (warp % 4)).
// One output tile [128 x BN] per CTA, STAGES-deep ring of K blocks (64 bf16 = one swizzle row).
// Out-of-range rows/columns are zero-filled by TMA on load and predicated on store, so any
// m >= 1 and n >= 1 work (decode batches of 1..64 rows, n = 50257 for the lm_head).
//
// All mbarrier waits are bounded; on expiry a status word is set and the CTA unwinds through the
// common exit that frees its TMEM columns.
#include "kernels.h"
#include "tma.h"

#include <cooperative_groups.h>
namespace cg = cooperative_groups;

namespace ak {

__device__ unsigned int g_gemm_status = 0;

constexpr int GB_M = 128;        // rows per tile (UMMA M)
constexpr int GB_K = 64;         // bf16 per K block = 128 bytes
constexpr int G_THREADS = 192;

// ---- tcgen05 wrappers ----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread i gets row (lane base + i), columns c..c+15.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle, rows of 128 bytes:
// 8-row atoms are 1024 bytes apart (stride byte offset), leading offset unused for this mode.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                        // leading byte offset (ignored), bits [16,30)
    d |= (uint64_t)(1024u >> 4) << 32;             // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                        // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                        // layout: SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16: D = f32, A = B = bf16, both K-major, shape M x N.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

constexpr int G_MAX_STAGES = 12;

// Cluster-wide barrier for all threads of all CTAs of the cluster. The .aligned forms need every
// thread of a warp to execute them together, and the producer / MMA lanes run ahead of their
// warps, so each warp is re-converged first.
__device__ __forceinline__ void cluster_arrive_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_all() {
    __syncwarp();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    cluster_arrive_all();
    cluster_wait_all();
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// 16 bytes into a peer CTA's shared memory; on arrival they are counted (complete_tx) on a barrier of that CTA
__device__ __forceinline__ void st_async_v4(uint32_t dst_cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t bar_cluster_addr) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(dst_cluster_addr),
                 "r"(a), "r"(b), "r"(c), "r"(d), "r"(bar_cluster_addr)
                 : "memory");
}

template <int BN> struct GemmCfg {
    static constexpr int B_BYTES = BN * GB_K * 2;   // weight tile of a stage; a multiple of 1024 for every BN % 8 == 0
};

// Epilogue arguments (by value).
struct GemmEpi {
    void* c;            // output matrix (f32 or bf16), may be null for the argmax-only epilogue
    uint32_t ldc;
    float* amax_val;    // [m][amax_ld] per-tile row maxima (argmax epilogues)
    uint32_t* amax_idx; // [m][amax_ld] their column indices
    uint32_t amax_ld;
};

enum { EPI_ARGMAX = 4, EPI_STORE_F32_ARGMAX = 5 };

// Store W consecutive accumulator columns of one row with the epilogue op. gcol % 4 == 0.
template <int EPI, int W>
__device__ __forceinline__ void epi_store(const GemmEpi& ep, uint32_t row, uint32_t gcol, const float* v, uint32_t n) {
    if (EPI == AK_EPI_STORE_F32 || EPI == AK_EPI_ADD_F32 || EPI == EPI_STORE_F32_ARGMAX) {
        float* dst = reinterpret_cast<float*>(ep.c) + (size_t)row * ep.ldc + gcol;
        const bool vec = (gcol + W <= n) && ((ep.ldc & 3u) == 0);
        if (vec) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (EPI == AK_EPI_ADD_F32) {
                    float4 p = *reinterpret_cast<float4*>(dst + j);
                    o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                *reinterpret_cast<float4*>(dst + j) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < W; j++)
                if (gcol + j < n) {
                    float o = v[j];
                    if (EPI == AK_EPI_ADD_F32) o += dst[j];
                    dst[j] = o;
                }
        }
    } else if (EPI == AK_EPI_STORE_BF16 || EPI == AK_EPI_SILU_BF16) {
        bf16* dst = reinterpret_cast<bf16*>(ep.c) + (size_t)row * ep.ldc + gcol;
        float t[W];
#pragma unroll
        for (int j = 0; j < W; j++) t[j] = (EPI == AK_EPI_SILU_BF16) ? v[j] / (1.0f + __expf(-v[j])) : v[j];
        const bool vec = (gcol + W <= n) && ((ep.ldc & 3u) == 0);
        if (W % 8 == 0 && vec && (ep.ldc & 7u) == 0 && (gcol & 7u) == 0) {
            // 16-byte stores: half as many L2 write requests per 32-byte sector as 8-byte ones
#pragma unroll
            for (int j = 0; j < W; j += 8) {
                uint32_t pk[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    bf162 a = __floats2bfloat162_rn(t[j + 2 * e], t[j + 2 * e + 1]);
                    pk[e] = *reinterpret_cast<uint32_t*>(&a);
                }
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        } else if (vec) {
#pragma unroll
            for (int j = 0; j < W; j += 4) {
                bf162 a = __floats2bfloat162_rn(t[j], t[j + 1]), b = __floats2bfloat162_rn(t[j + 2], t[j + 3]);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&a);
                pk.y = *reinterpret_cast<uint32_t*>(&b);
                *reinterpret_cast<uint2*>(dst + j) = pk;
            }
        } else {
#pragma unroll
            for (int j = 0; j < W; j++)
                if (gcol + j < n) dst[j] = __float2bfloat16_rn(t[j]);
        }
    }
}

// The 16-column form used by the one-CTA-per-tile epilogue, called by whole warps. A thread owns one
// row; its 16 columns are 64 bytes of f32 (two 32-byte sectors) or 32 bytes of bf16 (one sector).
// Writing them with 16-byte stores costs L2 two write requests per sector, and large-m launches are
// bound by exactly that. So adjacent lanes (rows r, r^1) trade halves: in one instruction the even
// lane covers the first 16 bytes of a sector and the odd lane the second, first for the even row,
// then for the odd row. Same number of instructions, every request a full sector.
template <int EPI>
__device__ __forceinline__ void epi_store16(const GemmEpi& ep, uint32_t row, bool row_ok, uint32_t gcol, const float* v, uint32_t n,
                                            uint32_t lane) {
    constexpr bool is_f32 = (EPI == AK_EPI_STORE_F32 || EPI == AK_EPI_ADD_F32 || EPI == EPI_STORE_F32_ARGMAX);
    const bool fast = (gcol + 16 <= n) && ((gcol & 7u) == 0) && ((ep.ldc & 7u) == 0) && ep.c != nullptr;  // warp-uniform
    if (!fast) {
        if (row_ok && ep.c != nullptr) epi_store<EPI, 16>(ep, row, gcol, v, n);
        return;
    }
    const bool odd = lane & 1u;
    const bool partner_ok = __shfl_xor_sync(0xffffffffu, row_ok ? 1 : 0, 1) != 0;
    const bool ok_a = odd ? partner_ok : row_ok, ok_b = odd ? row_ok : partner_ok;  // even row / odd row of the pair
    const uint32_t ra = row & ~1u;
    if (is_f32) {
        float* base_a = reinterpret_cast<float*>(ep.c) + (size_t)ra * ep.ldc + gcol + (odd ? 4 : 0);
        float* base_b = base_a + ep.ldc;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float own[4], got[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                own[e] = odd ? v[8 * i + 4 + e] : v[8 * i + e];
                const float send = odd ? v[8 * i + e] : v[8 * i + 4 + e];
                got[e] = __shfl_xor_sync(0xffffffffu, send, 1);
            }
            float4 xa = odd ? make_float4(got[0], got[1], got[2], got[3]) : make_float4(own[0], own[1], own[2], own[3]);
            float4 xb = odd ? make_float4(own[0], own[1], own[2], own[3]) : make_float4(got[0], got[1], got[2], got[3]);
            if (EPI == AK_EPI_ADD_F32) {
                float4 pa = make_float4(0.f, 0.f, 0.f, 0.f), pb = pa;
                if (ok_a) pa = *reinterpret_cast<const float4*>(base_a + 8 * i);
                if (ok_b) pb = *reinterpret_cast<const float4*>(base_b + 8 * i);
                xa.x += pa.x; xa.y += pa.y; xa.z += pa.z; xa.w += pa.w;
                xb.x += pb.x; xb.y += pb.y; xb.z += pb.z; xb.w += pb.w;
            }
            if (ok_a) *reinterpret_cast<float4*>(base_a + 8 * i) = xa;
            if (ok_b) *reinterpret_cast<float4*>(base_b + 8 * i) = xb;
        }
    } else {
        uint32_t pk[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float t0 = (EPI == AK_EPI_SILU_BF16) ? v[2 * e] / (1.0f + __expf(-v[2 * e])) : v[2 * e];
            const float t1 = (EPI == AK_EPI_SILU_BF16) ? v[2 * e + 1] / (1.0f + __expf(-v[2 * e + 1])) : v[2 * e + 1];
            bf162 a = __floats2bfloat162_rn(t0, t1);
            pk[e] = *reinterpret_cast<uint32_t*>(&a);
        }
        uint32_t got[4];
#pragma unroll
        for (int e = 0; e < 4; e++) got[e] = __shfl_xor_sync(0xffffffffu, odd ? pk[e] : pk[4 + e], 1);
        bf16* base_a = reinterpret_cast<bf16*>(ep.c) + (size_t)ra * ep.ldc + gcol + (odd ? 8 : 0);
        bf16* base_b = base_a + ep.ldc;
        const uint4 own = odd ? make_uint4(pk[4], pk[5], pk[6], pk[7]) : make_uint4(pk[0], pk[1], pk[2], pk[3]);
        const uint4 oth = make_uint4(got[0], got[1], got[2], got[3]);
        if (ok_a) *reinterpret_cast<uint4*>(base_a) = odd ? oth : own;
        if (ok_b) *reinterpret_cast<uint4*>(base_b) = odd ? own : oth;
    }
}

// Kernel. grid = (n tiles, m tiles, ks); thread-block cluster = (1, 1, ks): the ks CTAs of a
// cluster split the K range of ONE output tile, exchange their partial accumulators through
// distributed shared memory (every CTA receives the column slice it owns from every peer) and
// each reduces and stores its own slice in a fixed source order, so the result does not depend on
// timing. ks == 1 is the plain one-CTA-per-tile GEMM.
// SPLIT selects, at compile time, the cluster exchange epilogue (true) or the one-CTA-per-tile epilogue
// (false): a decode step is a chain of short launches whose first wave also pays for fetching the kernel's
// instructions, so each instantiation carries only the path it runs.
template <int BN, int EPI, bool SPLIT>
__global__ void __launch_bounds__(G_THREADS)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmEpi ep,
                 uint32_t m, uint32_t n, uint32_t k, uint32_t stages, uint32_t kseg, uint32_t tmem_cols, uint32_t a_rows) {
    // a_rows: rows of the activation box (128, or fewer when m is small: the MMA still reads 128 rows of
    // the stage, the rows past the box hold stale data and feed accumulator rows that are never stored).
    // kseg > 1 (only with a cluster of one CTA): the K range is accumulated in kseg separate TMEM
    // accumulators that the epilogue adds in order. It reproduces, bit for bit, what a cluster of
    // kseg CTAs computes for the same (n, k), so a row's result does not depend on how many rows
    // share the launch.
    using C = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[G_MAX_STAGES], empty_bar[G_MAX_STAGES], acc_bar, xch_bar;
    __shared__ uint32_t tmem_base_sm;
    __shared__ uint32_t fail_flag;

    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t ks = SPLIT ? cluster.num_blocks() : 1u;
    const uint32_t rank = SPLIT ? cluster.block_rank() : 0u;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // The ring: `stages` activation slots of a_rows x 128 B, then `stages` weight slots of BN x 128 B. A decode batch's
    // activation slot is as small as its TMA box, so the whole K range of a skinny CTA fits the ring and every weight
    // tile is requested before the dependency wait. The MMA still reads 128 rows from a slot's base: what follows it
    // (later slots, the weight slots, padding when those are too few) feeds accumulator rows that are never stored.
    // The split-K exchange buffer holds a_rows rows per source CTA (rows past m are never exchanged).
    const uint32_t a_bytes = a_rows * (GB_K * 2), stage_tx = a_bytes + C::B_BYTES;
    uint8_t* const b_base = smem + (size_t)stages * a_bytes;
    const uint32_t overrun = (GB_M - a_rows) * (GB_K * 2), b_total = stages * C::B_BYTES;
    float* red = reinterpret_cast<float*>(b_base + b_total + (overrun > b_total ? overrun - b_total : 0u));  // used when ks > 1
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m0 = blockIdx.y * GB_M, n0 = blockIdx.x * BN;
    const uint32_t num_kb_total = (k + GB_K - 1) / GB_K;
    const uint32_t per = (num_kb_total + ks - 1) / ks;
    const uint32_t kb_begin = rank * per < num_kb_total ? rank * per : num_kb_total;
    const uint32_t num_kb = (kb_begin + per <= num_kb_total) ? per : num_kb_total - kb_begin;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        mbar_init(&xch_bar, 1);
        fail_flag = 0;
        mbar_fence_init();
        if (SPLIT) {
            // the partial slices the peers will push into this CTA's exchange buffer: SL columns of every valid row
            // from each of the other ks - 1 CTAs (armed before the start barrier below, which the peers pass first)
            const uint32_t rows_here = (m - m0 < (uint32_t)GB_M) ? m - m0 : (uint32_t)GB_M;
            mbar_expect_tx(&xch_bar, (ks - 1) * rows_here * ((uint32_t)BN / ks) * 4u);
        }
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_sm, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    // "Every CTA of the cluster is running" must hold before anyone writes into a peer's shared
    // memory. Arrive now, wait only right before the exchange: the barrier latency hides behind
    // the main loop.
    __syncthreads();
    if (SPLIT) cluster_arrive_all();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_sm;
    // Everything above touched only this CTA's shared memory and TMEM. Let the next kernel's blocks
    // be scheduled as SMs free up; they, like this one, wait for their prerequisite grid before
    // touching anything it wrote.
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            // The weight tiles do not depend on the preceding kernel: the first ring of them is
            // requested BEFORE waiting for it, so the weight stream from HBM overlaps the
            // predecessor's tail. The activation tiles follow after the wait.
            const uint32_t pre = num_kb < stages ? num_kb : stages;
            for (uint32_t i = 0; i < pre; i++) {
                uint8_t* b_dst = b_base + (size_t)i * C::B_BYTES;
                mbar_expect_tx(&full_bar[i], stage_tx);
                tma_load_2d(b_dst, &tmB, (int32_t)((kb_begin + i) * GB_K), (int32_t)n0, &full_bar[i]);
            }
            pdl_wait();
            for (uint32_t i = 0; i < pre; i++)
                tma_load_2d(smem + (size_t)i * a_bytes, &tmA, (int32_t)((kb_begin + i) * GB_K), (int32_t)m0, &full_bar[i]);
            // ring position and phase are carried, not derived from i: an integer division costs this one thread
            // more than the four MMAs of a K block cost the tensor core
            uint32_t s = 0, ph = 1;   // i == pre == stages here: slot 0, second use
            for (uint32_t i = pre; i < num_kb; i++) {
                if (!mbar_wait(&empty_bar[s], ph ^ 1u)) { atomicExch(&fail_flag, 1u); break; }
                uint8_t* a_dst = smem + (size_t)s * a_bytes;
                uint8_t* b_dst = b_base + (size_t)s * C::B_BYTES;
                mbar_expect_tx(&full_bar[s], stage_tx);
                const int32_t kx = (int32_t)((kb_begin + i) * GB_K);
                tma_load_2d(a_dst, &tmA, kx, (int32_t)m0, &full_bar[s]);
                tma_load_2d(b_dst, &tmB, kx, (int32_t)n0, &full_bar[s]);
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(GB_M, BN);
            const uint32_t per_seg = (num_kb + kseg - 1) / kseg;
            uint32_t s = 0, ph = 0, in_seg = 0, acc_col = tmem_base;   // carried (no division in the loop, see the producer)
            for (uint32_t i = 0; i < num_kb; i++) {
                if (!mbar_wait(&full_bar[s], ph)) { atomicExch(&fail_flag, 2u); break; }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (size_t)s * a_bytes);
                const uint32_t b_addr = smem_u32(b_base + (size_t)s * C::B_BYTES);
                const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(b_addr);
#pragma unroll
                for (uint32_t kk = 0; kk < GB_K / 16; kk++) {
                    // advance 16 bf16 = 32 bytes along K inside the swizzle row: +2 in the address field
                    tc_mma_f16(acc_col, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (in_seg == 0 && kk == 0) ? 0u : 1u);
                }
                if (num_kb > stages) tc_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it (nobody waits when the ring holds the whole K range)
                if (++s == stages) { s = 0; ph ^= 1u; }
                if (++in_seg == per_seg) { in_seg = 0; acc_col += BN; }
            }
            if (num_kb > 0) tc_commit(&acc_bar);  // accumulator complete
            else mbar_arrive(&acc_bar);           // nothing to accumulate: this CTA contributes zeros
        }
    }

    // ---------------- epilogue warps 2..5: thread <-> accumulator row (TMEM lane)
    const uint32_t quad = warp & 3u;
    const uint32_t trow = quad * 32 + lane;  // row inside the tile
    const uint32_t row = m0 + trow;
    bool got = true, pre_ok = false;
    float4 pre0 = make_float4(0.f, 0.f, 0.f, 0.f), pre1 = pre0;
    if (warp >= 2) {
        pdl_wait();  // the epilogue reads and writes C: never before the preceding kernels are done
        if (SPLIT && EPI == AK_EPI_ADD_F32) {
            // the residual values this thread will add to: requested now, so that their L2 round trip runs under the
            // main loop and the exchange instead of after them
            const uint32_t SLp = (uint32_t)BN / ks, gc = n0 + rank * SLp;
            pre_ok = row < m && SLp <= 8 && (ep.ldc & 3u) == 0 && gc + SLp <= n;
            if (pre_ok) {
                const float* src = reinterpret_cast<const float*>(ep.c) + (size_t)row * ep.ldc + gc;
                pre0 = *reinterpret_cast<const float4*>(src);
                if (SLp == 8) pre1 = *reinterpret_cast<const float4*>(src + 4);
            }
        }
        got = mbar_wait(&acc_bar, 0);
        if (!got && lane == 0) atomicExch(&fail_flag, 3u);
        got = __all_sync(0xffffffffu, got);  // warp-uniform: TMEM loads and the paired stores below are warp-collective
        tc_fence_after();
    }

    if (!SPLIT) {
        if (warp >= 2 && got) {
            float best = -INFINITY;
            uint32_t best_i = 0xffffffffu;
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < (uint32_t)BN; c0 += 16) {
                uint32_t r[16];
                float v[16];
                if (num_kb > 0) {
                    tmem_ld16(tmem_base + ((quad * 32u) << 16) + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]);
                    for (uint32_t seg = 1; seg < kseg; seg++) {  // segment order = cluster rank order
                        tmem_ld16(tmem_base + ((quad * 32u) << 16) + seg * BN + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) v[j] += __uint_as_float(r[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = 0.0f;
                }
                if (EPI != EPI_ARGMAX) epi_store16<EPI>(ep, row, row < m, n0 + c0, v, n, lane);
                if (row < m) {
                    if (EPI == EPI_ARGMAX || EPI == EPI_STORE_F32_ARGMAX) {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (n0 + c0 + j < n && v[j] > best) { best = v[j]; best_i = n0 + c0 + j; }
                    }
                }
            }
            if ((EPI == EPI_ARGMAX || EPI == EPI_STORE_F32_ARGMAX) && row < m) {
                ep.amax_val[(size_t)row * ep.amax_ld + blockIdx.x] = best;
                ep.amax_idx[(size_t)row * ep.amax_ld + blockIdx.x] = best_i;
            }
        }
    } else {
        // ---- scatter: columns [d*SL, (d+1)*SL) of my partial go to CTA d's exchange buffer slot `rank`
        const uint32_t SL = (uint32_t)BN / ks;  // multiple of 4 by construction of the launch
        cluster_wait_all();  // phase 1: all peers are up (arrived at kernel start)
        if (warp >= 2 && got) {  // warp-uniform: tcgen05.ld is a warp-wide (.aligned) instruction
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < (uint32_t)BN; c0 += 16) {
                uint32_t r[16];
                if (num_kb > 0) {
                    tmem_ld16(tmem_base + ((quad * 32u) << 16) + c0, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) r[j] = 0u;
                }
                if (row < m) {
#pragma unroll
                    for (uint32_t j = 0; j < 16; j += 4) {
                        const uint32_t col = c0 + j, dest = col / SL, off = col - dest * SL;
                        float* slot = red + ((size_t)rank * a_rows + trow) * SL + off;
                        if (dest == rank) {   // my own slice: read back by this same thread
                            *reinterpret_cast<uint4*>(slot) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                        } else {              // a peer's: an asynchronous store that is counted on the peer's exchange barrier
                            st_async_v4(map_to_cta(smem_u32(slot), dest), r[j], r[j + 1], r[j + 2], r[j + 3], map_to_cta(smem_u32(&xch_bar), dest));
                        }
                    }
                }
            }
        }
        // Every peer's slices for this CTA have landed when the exchange barrier's byte count is met: no cluster-wide
        // barrier (0.75 us). A CTA leaves only after it has received everything addressed to it, so nobody writes
        // into a CTA that is gone.
        if (warp >= 2 && got) {
            bool landed = mbar_wait(&xch_bar, 0);
            if (!landed && lane == 0) atomicExch(&fail_flag, 6u);
            got = __all_sync(0xffffffffu, landed);
        }
        if (warp >= 2 && got && row < m) {
#pragma unroll 1
            for (uint32_t j = 0; j < SL; j += 4) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (uint32_t src = 0; src < ks; src++) {  // fixed order: deterministic sum
                    float4 p = *reinterpret_cast<const float4*>(red + ((size_t)src * a_rows + trow) * SL + j);
                    acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
                }
                float v[4] = {acc.x, acc.y, acc.z, acc.w};
                if (EPI == AK_EPI_ADD_F32 && pre_ok) {
                    const float4 p = j == 0 ? pre0 : pre1;
                    v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
                    epi_store<AK_EPI_STORE_F32, 4>(ep, row, n0 + rank * SL + j, v, n);
                } else {
                    epi_store<EPI, 4>(ep, row, n0 + rank * SL + j, v, n);
                }
            }
        }
    }
    // ---------------- common exit
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && fail_flag) atomicExch(&g_gemm_status, fail_flag);
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair kernel for large m: tcgen05.mma.cta_group::2, persistent, double-buffered accumulators.
//
// A cluster of two CTAs (on the two SMs of a TPC; one CTA per SM, one pair per SM pair) walks over [256 x BN] output
// tiles. Each CTA stages ITS 128 rows of A and ITS half (BN/2 rows) of the weight tile per K block; the even CTA (the
// leader) issues one MMA of shape 256 x BN x 16 that reads both CTAs' shared memory and accumulates rows 0-127 into
// the leader's TMEM and rows 128-255 into the peer's. Per SM and K block that is 16 KB of A + BN/4 KB of B for a
// 128 x BN slice of output: half the weight traffic from L2 per flop of the one-CTA kernel, which is what bounds that
// kernel. The 512 TMEM columns hold TWO accumulator buffers: the epilogue warps drain tile i while the MMAs of tile
// i+1 run, so no second CTA per SM is needed to hide the epilogue and the ring can use the whole shared memory.
// Synchronisation (every wait bounded):
//   full[s]      leader's barrier; both CTAs' TMA loads (.cta_group::2, no multicast: each CTA fetches its own tiles)
//                complete on it, the leader arms it with the bytes of both;
//   empty[s]     one per CTA; after the MMAs of a K block the leader commits to its own and to the peer's
//                (two plain tcgen05.commit, the peer's addressed through the cluster window);
//   acc_full[b]  one per CTA, committed by the leader after a tile's last MMA;
//   acc_empty[b] leader's barrier, 8 arrivals: one per epilogue warp of both CTAs (the peer's arrive remotely).
// TMEM is allocated and freed with the .cta_group::2 forms by warp 1 of both CTAs, with cluster barriers after the
// allocation and before the release.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the mbarrier at shared::cluster address `bar_cluster_addr` once every MMA issued so far has completed
__device__ __forceinline__ void tc_commit2(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_mma2_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// TMA tiled load of a CTA pair: the data lands in THIS CTA's shared memory, the bytes are counted on the mbarrier at
// `bar_cluster_addr`, which may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, int32_t x, int32_t y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

template <int BN> struct PairCfg {
    static constexpr int A_BYTES = GB_M * GB_K * 2;          // this CTA's 128 rows of A: 16 KB
    static constexpr int B_BYTES = (BN / 2) * GB_K * 2;      // this CTA's half of the weight tile
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = 512;                    // two accumulator buffers of kseg * BN columns
};

template <int BN, int EPI>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmEpi ep,
                      uint32_t m, uint32_t n, uint32_t k, uint32_t stages, uint32_t kseg, uint32_t tiles_n, uint32_t tiles_total) {
    using C = PairCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[G_MAX_STAGES], empty_bar[G_MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_sm;
    __shared__ uint32_t fail_flag;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs), 1 = peer
    const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t num_kb = (k + GB_K - 1) / GB_K;
    const uint32_t buf_cols = kseg * BN;
    // two accumulator buffers when they fit the 512 columns (the epilogue of a tile then runs under the next tile's
    // MMAs), else one (K split in two segments of 256 columns each: the epilogue is exposed)
    const uint32_t n_bufs = (2 * buf_cols <= (uint32_t)C::TMEM_COLS) ? 2u : 1u;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (uint32_t b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        fail_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc2(&tmem_base_sm, C::TMEM_COLS);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    // both CTAs hold their TMEM columns and have initialised their barriers before either touches the other's
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_sm;
    pdl_trigger();   // only after the TMEM allocation (see the one-CTA kernel)

    if (warp == 0) {
        // ---------------- TMA producer (one per CTA; bytes are counted on the leader's full barriers)
        if (lane == 0) {
            pdl_wait();
            uint32_t it = 0, s = 0, ph = 0;   // ring position and phase are carried: no division in the K loop
            bool ok = true;
            for (uint32_t t = pair; t < tiles_total && ok; t += n_pairs) {
                const uint32_t m0 = ((t / tiles_n) * 2 + rank) * GB_M;        // this CTA's 128 rows of the pair's 256
                const uint32_t nb0 = (t % tiles_n) * BN + rank * (BN / 2);    // this CTA's half of the weight rows
                for (uint32_t kb = 0; kb < num_kb; kb++, it++) {
                    if (it >= stages && !mbar_wait(&empty_bar[s], ph ^ 1u)) { atomicExch(&fail_flag, 1u); ok = false; break; }
                    uint8_t* a_dst = smem + (size_t)s * C::STAGE_BYTES;
                    const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);
                    const int32_t kx = (int32_t)(kb * GB_K);
                    tma_load_2d_pair(a_dst, &tmA, kx, (int32_t)m0, bar);
                    tma_load_2d_pair(a_dst + C::A_BYTES, &tmB, kx, (int32_t)nb0, bar);
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
            }
            // drain: every commit the leader addressed to this CTA's empty barriers has landed before the CTA may leave
            // (the last min(it, stages) uses, oldest first; with it >= stages the oldest one sits in slot s, the next to
            // be overwritten, one round behind the carried phase)
            if (ok && it > 0) {
                const bool wrapped = it >= stages;
                uint32_t ds = wrapped ? s : 0u, dph = wrapped ? (ph ^ 1u) : 0u;
                const uint32_t cnt = wrapped ? stages : it;
                for (uint32_t j = 0; j < cnt; j++) {
                    if (!mbar_wait(&empty_bar[ds], dph)) { atomicExch(&fail_flag, 5u); break; }
                    if (++ds == stages) { ds = 0; dph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: one thread of the leader CTA drives both SMs' tensor cores
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc(2 * GB_M, BN);
            const uint32_t per_seg = (num_kb + kseg - 1) / kseg;
            uint32_t tc = 0, s = 0, ph = 0;   // ring position and phase are carried: no division in the K loop
            bool ok = true;
            for (uint32_t t = pair; t < tiles_total && ok; t += n_pairs, tc++) {
                const uint32_t buf = n_bufs == 2 ? (tc & 1u) : 0u, acc_ph = (n_bufs == 2 ? (tc >> 1) : tc) & 1u;
                // the epilogue warps of both CTAs have drained this buffer (it was last used by tile tc - n_bufs)
                if (tc >= n_bufs && !mbar_wait(&acc_empty[buf], acc_ph ^ 1u)) { atomicExch(&fail_flag, 4u); break; }
                tc_fence_after();
                uint32_t in_seg = 0, acc_col = tmem_base + buf * buf_cols;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&full_bar[s], ph)) { atomicExch(&fail_flag, 2u); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * C::STAGE_BYTES);
                    const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + C::A_BYTES);
#pragma unroll
                    for (uint32_t kk = 0; kk < GB_K / 16; kk++)
                        tc_mma2_f16(acc_col, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (in_seg == 0 && kk == 0) ? 0u : 1u);
                    // the stage is reusable in BOTH CTAs once these MMAs have read it
                    tc_commit2(map_to_cta(smem_u32(&empty_bar[s]), 0));
                    tc_commit2(map_to_cta(smem_u32(&empty_bar[s]), 1));
                    if (++s == stages) { s = 0; ph ^= 1u; }
                    if (++in_seg == per_seg) { in_seg = 0; acc_col += BN; }
                }
                if (!ok) break;
                tc_commit2(map_to_cta(smem_u32(&acc_full[buf]), 0));
                tc_commit2(map_to_cta(smem_u32(&acc_full[buf]), 1));
            }
        }
    } else {
        // ---------------- epilogue warps 2..5 of both CTAs: thread <-> accumulator row of THIS CTA's TMEM
        const uint32_t quad = warp & 3u;
        pdl_wait();
        uint32_t tc = 0;
        for (uint32_t t = pair; t < tiles_total; t += n_pairs, tc++) {
            const uint32_t buf = n_bufs == 2 ? (tc & 1u) : 0u, acc_ph = (n_bufs == 2 ? (tc >> 1) : tc) & 1u;
            const uint32_t row = ((t / tiles_n) * 2 + rank) * GB_M + quad * 32 + lane;
            const uint32_t n0 = (t % tiles_n) * BN;
            bool got = num_kb == 0 || mbar_wait(&acc_full[buf], acc_ph);
            if (!got && lane == 0) atomicExch(&fail_flag, 3u);
            got = __all_sync(0xffffffffu, got);
            if (!got) break;
            tc_fence_after();
            float best = -INFINITY;
            uint32_t best_i = 0xffffffffu;
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < (uint32_t)BN; c0 += 16) {
                uint32_t r[16];
                float v[16];
                if (num_kb > 0) {
                    tmem_ld16(tmem_base + ((quad * 32u) << 16) + buf * buf_cols + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]);
                    for (uint32_t seg = 1; seg < kseg; seg++) {
                        tmem_ld16(tmem_base + ((quad * 32u) << 16) + buf * buf_cols + seg * BN + c0, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) v[j] += __uint_as_float(r[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = 0.0f;
                }
                if (EPI != EPI_ARGMAX) epi_store16<EPI>(ep, row, row < m, n0 + c0, v, n, lane);
                if (row < m && (EPI == EPI_ARGMAX || EPI == EPI_STORE_F32_ARGMAX)) {
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (n0 + c0 + j < n && v[j] > best) { best = v[j]; best_i = n0 + c0 + j; }
                }
            }
            if ((EPI == EPI_ARGMAX || EPI == EPI_STORE_F32_ARGMAX) && row < m) {
                ep.amax_val[(size_t)row * ep.amax_ld + (t % tiles_n)] = best;
                ep.amax_idx[(size_t)row * ep.amax_ld + (t % tiles_n)] = best_i;
            }
            // this warp has read its part of the buffer: let the leader's MMA thread reuse it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
        }
    }
    // ---------------- common exit: nobody frees TMEM or leaves while the pair may still use this CTA's memory
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && fail_flag) atomicExch(&g_gemm_status, fail_flag);
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc2(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// Launch configuration.
struct GemmPlan {
    uint32_t bn, ks, stages;
    uint32_t kseg;  // in-CTA K segments (large m with invariant = true), else 1
};

static constexpr uint32_t SMEM_TWO_PER_SM = 112 * 1024;   // two CTAs fit one SM below this
static constexpr uint32_t SMEM_ONE_PER_SM = 220 * 1024;
static constexpr uint32_t SMEM_THREE_PER_SM = 74 * 1024;  // three CTAs fit one SM below this (228 KB, 1 KB reserved and ~0.25 KB static per CTA)

// Rows of the activation TMA box: a decode batch fills only part of the 128-row MMA tile, and rows the
// box does not fetch cost neither L2 requests nor zero-fill writes.
static uint32_t a_box_rows(uint32_t m) {
    if (m > 64) return GB_M;
    return m > 32 ? 64 : (m > 16 ? 32 : 16);
}
static uint32_t stage_bytes(uint32_t bn, uint32_t a_rows = GB_M) { return a_rows * GB_K * 2 + bn * GB_K * 2; }
// shared memory of the one-CTA kernel: the ring, the rows an MMA reads past a short activation slot where the weight
// slots do not cover them, the exchange buffer (a_rows rows per source CTA), alignment room
static size_t gemm_smem_bytes(uint32_t stages, uint32_t bn, uint32_t a_rows, bool split) {
    const size_t overrun = (size_t)(GB_M - a_rows) * GB_K * 2, b_total = (size_t)stages * bn * GB_K * 2;
    return (size_t)stages * stage_bytes(bn, a_rows) + (overrun > b_total ? overrun - b_total : 0) + (split ? (size_t)a_rows * bn * 4 : 0) + 1024;
}
// most stages (<= want) whose ring, exchange buffer and padding fit `budget` bytes
static uint32_t gemm_fit_stages(uint32_t want, uint32_t bn, uint32_t a_rows, bool split, uint32_t budget) {
    uint32_t st = want > G_MAX_STAGES ? G_MAX_STAGES : want;
    while (st > 1 && gemm_smem_bytes(st, bn, a_rows, split) > budget) st--;
    return st;
}

// Skinny problems (m <= 128: decode batches) are latency- and weight-stream-bound: pick the
// tile width / K split that gives one wave of up to 296 CTAs (two per SM) with the shortest K
// chain per CTA. Large m uses wide tiles and deep pipelines.
static GemmPlan plan_gemm(uint32_t m, uint32_t n, uint32_t k, bool allow_split, bool invariant = false) {
    const uint32_t num_kb = cdiv(k, GB_K);
    GemmPlan p{};
    p.kseg = 1;
    if (m > GB_M && invariant && allow_split) {
        // same K partition as the skinny plan of this (n, k)
        const GemmPlan sk = plan_gemm(GB_M, n, k, true, false);
        if (sk.ks > 1) {
            const uint32_t mt = cdiv(m, GB_M);
            if (mt <= 4 && sk.ks == 2) {
                // qkv / ffn-up with a prompt or two beside the decode rows: the two K halves as two accumulators
                // of one CTA (same summation structure as the 2-CTA cluster exchange of the decode plan, without
                // the exchange); measured 3-6 % off an admission step against the cluster form
                p.kseg = 2; p.ks = 1; p.bn = 64;
                uint32_t st = (SMEM_THREE_PER_SM - 1024) / stage_bytes(p.bn);   // three per SM: these run beside the decode rows' chain
                if (st > G_MAX_STAGES) st = G_MAX_STAGES;
                p.stages = st < num_kb ? st : num_kb;
                return p;
            }
            if (mt <= 4) {
                // A prompt or two joining a decode batch: the K chain per CTA, not the flop count, sets the
                // time (an MMA of 64 columns or fewer costs the same ~50 cycles), so keep the cluster split of
                // the decode plan, with the widest tile that still fits one wave of two CTAs per SM.
                p.ks = sk.ks;
                p.bn = 16;
                const uint32_t cands[3] = {64, 32, 16};   // measured: starting from 32 or 16 is slower (1.23 / 1.28 ms against 1.14)
                for (int i = 0; i < 3; i++)
                    if ((cands[i] / p.ks) % 4 == 0 && (uint64_t)mt * cdiv(n, cands[i]) * p.ks <= 296) { p.bn = cands[i]; break; }
                if ((p.bn / p.ks) % 4 != 0) p.bn = 4 * p.ks;  // 16 or 32: always a legal tile width
                const uint32_t per = cdiv(num_kb, p.ks);
                uint32_t st = gemm_fit_stages(per ? per : 1, p.bn, GB_M, true, SMEM_TWO_PER_SM);
                if (st < 2 && per >= 2) st = 2;
                p.stages = st;
                return p;
            }
            p.kseg = sk.ks;
            p.ks = 1;
            // widest tile whose accumulators fit TMEM (kseg * bn <= 512 columns); narrower while
            // the grid would leave most SMs idle
            p.bn = 512 / sk.ks > 256 ? 256 : 512 / sk.ks;
            while (p.bn > 32 && (uint64_t)mt * cdiv(n, p.bn) < B200_SMS) p.bn /= 2;
            uint32_t st = (SMEM_ONE_PER_SM - 1024) / stage_bytes(p.bn);
            if (st > G_MAX_STAGES) st = G_MAX_STAGES;
            if (p.bn <= 64 && st > 6) st = 6;
            p.stages = st < num_kb ? st : num_kb;
            return p;
        }
    }
    if (m > GB_M) {
        const uint32_t mt = cdiv(m, GB_M);
        const uint32_t cands[5] = {256, 128, 64, 32, 16};
        p.bn = 16;
        for (int i = 0; i < 5; i++)
            if ((uint64_t)mt * cdiv(n, cands[i]) >= B200_SMS) { p.bn = cands[i]; break; }
        p.ks = 1;
        // Two CTAs per SM (one's epilogue under the other's main loop) beat one CTA with a deeper ring.
        uint32_t st = (SMEM_TWO_PER_SM - 1024) / stage_bytes(p.bn);
        if (st > G_MAX_STAGES) st = G_MAX_STAGES;
        if (p.bn <= 64 && st > 6) st = 6;
        p.stages = st < num_kb ? st : (num_kb ? num_kb : 1);
        return p;
    }
    const uint32_t slots = 296;
    if (cdiv(n, 64) > slots) {
        // very wide n (the lm_head): one wave of wide tiles, two CTAs per SM
        const uint32_t cands[3] = {128, 176, 256};
        p.bn = 256;
        for (int i = 0; i < 3; i++)
            if (cdiv(n, cands[i]) <= slots) { p.bn = cands[i]; break; }
        p.ks = 1;
        const uint32_t ar = a_box_rows(m);
        uint32_t st = (SMEM_TWO_PER_SM - 1024 - (GB_M - ar) * GB_K * 2) / stage_bytes(p.bn, ar);
        if (st > G_MAX_STAGES) st = G_MAX_STAGES;
        if (st < 2) st = 2;
        p.stages = st < num_kb ? st : (num_kb ? num_kb : 1);
        return p;
    }
    uint32_t best_kb = 0xffffffffu, best_ctas = 0;
    p = GemmPlan{16, 1, 1, 1};
    const uint32_t bns[3] = {16, 32, 64};
    const uint32_t kss[4] = {1, 2, 4, 8};
    for (int bi = 0; bi < 3; bi++)
        for (int ki = 0; ki < 4; ki++) {
            const uint32_t bn = bns[bi], ks = kss[ki];
            // One MMA (M = 128 or 64, K = 16) occupies the tensor core 50 cycles for any N <= 64 (64 cycles at
            // N = 128, 128 at N = 256), and the issuing thread needs ~0.2 us per K block (wait, four MMAs, commit),
            // so a CTA's main loop costs the same however narrow its tile; a cluster exchange costs ~1.2 us, the
            // boundary to the next launch ~2 us. Split long K chains (K > 1024), and
            // short ones four ways only when the unsplit grid would cover less than half of the SMs.
            // Other short chains are halved at most (two accumulators still leave 256-column tiles to
            // the large-m plan) and only with tiles of 32 columns or more per exchange.
            const bool short_k_ok = cdiv(n, 16) * 2 <= B200_SMS;
            if (ks > 1 && num_kb <= 16 && !short_k_ok && (ks > 2 || bn < 32)) continue;
            if (ks > 1 && (!allow_split || ks * 2 > num_kb || (bn / ks) % 4 != 0)) continue;
            const uint32_t per = cdiv(num_kb, ks);
            if (ks > 1 && (ks - 1) * per >= num_kb) continue;  // every CTA of the cluster gets work
            const uint32_t ctas = cdiv(n, bn) * ks;
            if (ctas > slots && !(bi == 2 && ki == 0)) continue;
            const bool better = per < best_kb || (per == best_kb && ctas > best_ctas);   // more, narrower CTAs measured faster than one wide wave
            if (better) { best_kb = per; best_ctas = ctas; p.bn = bn; p.ks = ks; }
        }
    const uint32_t per = cdiv(num_kb, p.ks) ? cdiv(num_kb, p.ks) : 1;
    const uint32_t ar = a_box_rows(m);
    uint32_t st = gemm_fit_stages(per, p.bn, ar, p.ks > 1, SMEM_TWO_PER_SM);
    // A footprint that lets THREE CTAs share an SM is preferred when it costs at most one stage of the K range (that
    // K block then re-uses the first slot): the next launch's CTAs, and the attention CTAs behind the qkv projection,
    // find room on every SM while this launch still runs. Measured on the 162M decode step: 0.552 ms against 0.562 ms
    // with the whole K range resident at two CTAs per SM (and 0.587 ms with this ring layout at two per SM).
    const uint32_t st3 = gemm_fit_stages(per, p.bn, ar, p.ks > 1, SMEM_THREE_PER_SM);
    if (st3 + 1 >= per && st3 >= 2) st = st3;
    if (st < 2 && per >= 2) st = 2;
    p.stages = st;
    return p;
}

template <int BN, int EPI>
static int launch_cfg(cudaStream_t st, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmEpi& ep, uint32_t m, uint32_t n,
                      uint32_t k, const GemmPlan& p) {
    const size_t smem = gemm_smem_bytes(p.stages, BN, a_box_rows(m), p.ks > 1);
    {
        // per-device "attribute set" flags; the library may be driven from one host thread per GPU
        static size_t attr_set[64] = {};
        int dev = 0;
        AK_CUDA(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(device_cache_mutex());
        if (attr_set[dev & 63] < smem) {
            AK_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<BN, EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ONE_PER_SM));
            AK_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<BN, EPI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ONE_PER_SM));
            attr_set[dev & 63] = SMEM_ONE_PER_SM;
        }
    }
    uint32_t need = p.kseg * BN, cols = 32;
    while (cols < need) cols *= 2;
    AK_REQUIRE(cols <= 512, AK_ERR_UNSUPPORTED, "gemm_bf16: %u accumulator columns exceed TMEM", need);
    if (p.ks > 1)
        return launch_k(gemm_bf16_kernel<BN, EPI, true>, dim3(cdiv(n, BN), cdiv(m, GB_M), p.ks), dim3(G_THREADS), smem, st, dim3(1, 1, p.ks),
                        tmA, tmB, ep, m, n, k, p.stages, p.kseg, cols, a_box_rows(m));
    return launch_k(gemm_bf16_kernel<BN, EPI, false>, dim3(cdiv(n, BN), cdiv(m, GB_M), 1), dim3(G_THREADS), smem, st, dim3(1, 1, 1),
                    tmA, tmB, ep, m, n, k, p.stages, p.kseg, cols, a_box_rows(m));
}

template <int BN>
static int launch_bn(cudaStream_t st, const void* a, const void* wt, const GemmEpi& ep, uint32_t m, uint32_t n, uint32_t k,
                     uint32_t epi, const GemmPlan& p) {
    CUtensorMap tmA, tmB;
    int rc = make_tmap_2d(&tmA, a, 2, k, m, (uint64_t)k * 2, GB_K, a_box_rows(m), TMA_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, wt, 2, k, n, (uint64_t)k * 2, GB_K, BN, TMA_SWIZZLE_128B);
    if (rc) return rc;
    switch (epi) {
        case AK_EPI_STORE_F32: return launch_cfg<BN, AK_EPI_STORE_F32>(st, tmA, tmB, ep, m, n, k, p);
        case AK_EPI_ADD_F32: return launch_cfg<BN, AK_EPI_ADD_F32>(st, tmA, tmB, ep, m, n, k, p);
        case AK_EPI_STORE_BF16: return launch_cfg<BN, AK_EPI_STORE_BF16>(st, tmA, tmB, ep, m, n, k, p);
        case AK_EPI_SILU_BF16: return launch_cfg<BN, AK_EPI_SILU_BF16>(st, tmA, tmB, ep, m, n, k, p);
        case EPI_ARGMAX: return launch_cfg<BN, EPI_ARGMAX>(st, tmA, tmB, ep, m, n, k, p);
        case EPI_STORE_F32_ARGMAX: return launch_cfg<BN, EPI_STORE_F32_ARGMAX>(st, tmA, tmB, ep, m, n, k, p);
    }
    set_error("gemm_bf16: unknown epilogue %u", epi);
    return AK_ERR_INVALID_ARG;
}

static int launch_planned(cudaStream_t st, const void* a, const void* wt, const GemmEpi& ep, uint32_t m, uint32_t n, uint32_t k,
                          uint32_t epi, const GemmPlan& p) {
    switch (p.bn) {
        case 256: return launch_bn<256>(st, a, wt, ep, m, n, k, epi, p);
        case 176: return launch_bn<176>(st, a, wt, ep, m, n, k, epi, p);
        case 128: return launch_bn<128>(st, a, wt, ep, m, n, k, epi, p);
        case 64: return launch_bn<64>(st, a, wt, ep, m, n, k, epi, p);
        case 32: return launch_bn<32>(st, a, wt, ep, m, n, k, epi, p);
        default: return launch_bn<16>(st, a, wt, ep, m, n, k, epi, p);
    }
}

// ---- the CTA-pair kernel's launch
template <int BN, int EPI>
static int launch_pair_cfg(cudaStream_t st, const void* a, const void* wt, const GemmEpi& ep, uint32_t m, uint32_t n, uint32_t k, uint32_t kseg) {
    using C = PairCfg<BN>;
    uint32_t stages = (SMEM_ONE_PER_SM - 1024) / C::STAGE_BYTES;
    if (stages > G_MAX_STAGES) stages = G_MAX_STAGES;
    const size_t smem = (size_t)stages * C::STAGE_BYTES + 1024;
    {
        static bool attr_set[64] = {};
        int dev = 0;
        AK_CUDA(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(device_cache_mutex());
        if (!attr_set[dev & 63]) {
            AK_CUDA(cudaFuncSetAttribute(gemm_bf16_pair_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ONE_PER_SM));
            attr_set[dev & 63] = true;
        }
    }
    CUtensorMap tmA, tmB;
    AK_TRY(make_tmap_2d(&tmA, a, 2, k, m, (uint64_t)k * 2, GB_K, GB_M, TMA_SWIZZLE_128B));
    AK_TRY(make_tmap_2d(&tmB, wt, 2, k, n, (uint64_t)k * 2, GB_K, BN / 2, TMA_SWIZZLE_128B));
    const uint32_t tiles_n = cdiv(n, BN), tiles_total = tiles_n * cdiv(m, 2 * GB_M);
    const uint32_t n_pairs = tiles_total < 74 ? tiles_total : 74;   // one pair per TPC of the 148 SMs
    return launch_k(gemm_bf16_pair_kernel<BN, EPI>, dim3(2 * n_pairs, 1, 1), dim3(G_THREADS), smem, st, dim3(2, 1, 1), tmA, tmB, ep, m, n, k,
                    stages, kseg, tiles_n, tiles_total);
}
template <int BN>
static int launch_pair(cudaStream_t st, const void* a, const void* wt, const GemmEpi& ep, uint32_t m, uint32_t n, uint32_t k, uint32_t epi,
                       uint32_t kseg) {
    switch (epi) {
        case AK_EPI_STORE_F32: return launch_pair_cfg<BN, AK_EPI_STORE_F32>(st, a, wt, ep, m, n, k, kseg);
        case AK_EPI_ADD_F32: return launch_pair_cfg<BN, AK_EPI_ADD_F32>(st, a, wt, ep, m, n, k, kseg);
        case AK_EPI_STORE_BF16: return launch_pair_cfg<BN, AK_EPI_STORE_BF16>(st, a, wt, ep, m, n, k, kseg);
        case AK_EPI_SILU_BF16: return launch_pair_cfg<BN, AK_EPI_SILU_BF16>(st, a, wt, ep, m, n, k, kseg);
    }
    set_error("gemm_bf16: unknown epilogue %u", epi);
    return AK_ERR_INVALID_ARG;
}
// Large m goes to the CTA-pair kernel when its K partition is a single accumulator of 256 columns (two TMEM
// buffers, the epilogue of a tile overlapped with the next tile's MMAs).
static bool pair_plan(uint32_t m, uint32_t n, uint32_t k, bool allow_split, bool invariant, uint32_t& bn, uint32_t& kseg) {
    if (m < 1024 || n < 256) return false;
    kseg = 1;
    if (invariant && allow_split) {
        // With K split in two segments of 256 columns the accumulators fill TMEM, the epilogue is exposed and the
        // kernel is no faster than the one-CTA kernel (measured on the 1.4B prefill: 12.0 s against 11.9 s): only
        // unsplit K partitions go to the pair kernel. (The kernel itself handles kseg = 2 with a single buffer.)
        const GemmPlan sk = plan_gemm(GB_M, n, k, true, false);
        if (sk.ks > 1) return false;
    }
    bn = 256;
    return true;
}

static int check_operands(const void* a, const void* wt, uint32_t k) {
    AK_REQUIRE(k >= 8 && k % 8 == 0, AK_ERR_UNSUPPORTED, "gemm_bf16: k (%u) must be a positive multiple of 8", k);
    AK_REQUIRE(((uintptr_t)a % 16) == 0 && ((uintptr_t)wt % 16) == 0, AK_ERR_INVALID_ARG, "gemm_bf16: operands must be 16-byte aligned");
    return AK_OK;
}

int launch_gemm_bf16(cudaStream_t st, const void* a, const void* wt, void* c, uint32_t m, uint32_t n, uint32_t k,
                     uint32_t epilogue, uint32_t ldc, bool invariant) {
    if (m == 0 || n == 0) return AK_OK;
    int rc = check_operands(a, wt, k);
    if (rc) return rc;
    AK_REQUIRE(epilogue <= AK_EPI_SILU_BF16, AK_ERR_INVALID_ARG, "gemm_bf16: unknown epilogue %u", epilogue);
    AK_REQUIRE(((uintptr_t)c % 16) == 0, AK_ERR_INVALID_ARG, "gemm_bf16: output must be 16-byte aligned");
    GemmEpi ep{};
    ep.c = c;
    ep.ldc = ldc ? ldc : n;
    // the split-K exchange stores 4-column groups: it needs 4-aligned rows
    const bool allow_split = (ep.ldc % 4) == 0;
    uint32_t pbn = 0, pkseg = 1;
    if (pair_plan(m, n, k, allow_split, invariant, pbn, pkseg)) return launch_pair<256>(st, a, wt, ep, m, n, k, epilogue, pkseg);
    return launch_planned(st, a, wt, ep, m, n, k, epilogue, plan_gemm(m, n, k, allow_split, invariant));
}

uint32_t gemm_argmax_tiles(uint32_t m, uint32_t n, uint32_t k) { return cdiv(n, plan_gemm(m, n, k, false).bn); }

// logits (optional, f32 [m, ldc]) and per-tile row maxima; a second tiny kernel finishes the argmax.
int launch_gemm_bf16_argmax(cudaStream_t st, const void* a, const void* wt, float* logits, uint32_t ldc, float* part_val,
                            uint32_t* part_idx, uint32_t m, uint32_t n, uint32_t k) {
    if (m == 0 || n == 0) return AK_OK;
    int rc = check_operands(a, wt, k);
    if (rc) return rc;
    GemmPlan p = plan_gemm(m, n, k, false);
    p.ks = 1;
    GemmEpi ep{};
    ep.c = logits;
    ep.ldc = ldc ? ldc : n;
    ep.amax_val = part_val;
    ep.amax_idx = part_idx;
    ep.amax_ld = cdiv(n, p.bn);
    return launch_planned(st, a, wt, ep, m, n, k, logits ? EPI_STORE_F32_ARGMAX : EPI_ARGMAX, p);
}

int gemm_bf16_check_status(cudaStream_t st) {
    AK_CUDA(cudaStreamSynchronize(st));
    unsigned int v = 0;
    AK_CUDA(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(v)));
    AK_REQUIRE(v == 0, AK_ERR_DEVICE_WAIT, "gemm_bf16: a bounded device-side wait expired (code %u)", v);
    return AK_OK;
}

}  // namespace ak

using namespace ak;
extern "C" int ak_gemm_bf16(void* stream, const void* a, const void* wt, void* c, ak_matmul_meta m, uint32_t epilogue) {
    AK_REQUIRE(a && wt && c, AK_ERR_INVALID_ARG, "ak_gemm_bf16: null pointer");
    return launch_gemm_bf16(as_stream(stream), a, wt, c, m.m, m.n, m.k, epilogue, m.n, false);
}
extern "C" int ak_gemm_bf16_ld(void* stream, const void* a, const void* wt, void* c, ak_matmul_meta m, uint32_t epilogue, uint32_t ldc) {
    AK_REQUIRE(a && wt && c, AK_ERR_INVALID_ARG, "ak_gemm_bf16_ld: null pointer");
    AK_REQUIRE(ldc >= m.n, AK_ERR_INVALID_ARG, "ak_gemm_bf16_ld: ldc (%u) must be at least n (%u)", ldc, m.n);
    return launch_gemm_bf16(as_stream(stream), a, wt, c, m.m, m.n, m.k, epilogue, ldc, false);
}

