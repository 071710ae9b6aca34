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

template <int BN> struct GemmCfg {
    static constexpr int A_BYTES = GB_M * GB_K * 2;   // 16 KB
    static constexpr int B_BYTES = BN * GB_K * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
};

template <int BN, int EPI>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ cptr,
                 uint32_t m, uint32_t n, uint32_t k, uint32_t ldc) {
    using C = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[C::STAGES], empty_bar[C::STAGES], acc_bar;
    __shared__ uint32_t tmem_base_sm;
    __shared__ uint32_t fail_flag;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m0 = blockIdx.y * GB_M, n0 = blockIdx.x * BN;
    const uint32_t num_kb = (k + GB_K - 1) / GB_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        fail_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_sm, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_sm;

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            for (uint32_t kb = 0; kb < num_kb; kb++) {
                const uint32_t s = kb % C::STAGES, ph = (kb / C::STAGES) & 1u;
                if (!mbar_wait(&empty_bar[s], ph ^ 1u)) { atomicExch(&fail_flag, 1u); break; }
                uint8_t* a_dst = smem + (size_t)s * C::STAGE_BYTES;
                uint8_t* b_dst = a_dst + C::A_BYTES;
                mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                tma_load_2d(a_dst, &tmA, (int32_t)(kb * GB_K), (int32_t)m0, &full_bar[s]);
                tma_load_2d(b_dst, &tmB, (int32_t)(kb * GB_K), (int32_t)n0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(GB_M, BN);
            bool ok = true;
            for (uint32_t kb = 0; kb < num_kb && ok; kb++) {
                const uint32_t s = kb % C::STAGES, ph = (kb / C::STAGES) & 1u;
                if (!mbar_wait(&full_bar[s], ph)) { atomicExch(&fail_flag, 2u); ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (size_t)s * C::STAGE_BYTES);
                const uint32_t b_addr = a_addr + C::A_BYTES;
                const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(b_addr);
#pragma unroll
                for (uint32_t kk = 0; kk < GB_K / 16; kk++) {
                    // advance 16 bf16 = 32 bytes along K inside the swizzle row: +2 in the address field
                    tc_mma_f16(tmem_base, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb | kk) != 0 ? 1u : 0u);
                }
                tc_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it
            }
            tc_commit(&acc_bar);           // accumulator complete
        }
    } else {
        // ---------------- epilogue warps 2..5
        const uint32_t quad = warp & 3u;  // TMEM lanes [32*quad, 32*quad+32)
        const bool got = mbar_wait(&acc_bar, 0);
        if (!got && lane == 0) atomicExch(&fail_flag, 3u);
        tc_fence_after();
        const uint32_t row = m0 + quad * 32 + lane;
        if (got && num_kb > 0) {
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < (uint32_t)BN; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem_base + ((quad * 32u) << 16) + c0, r);
                tmem_ld_wait();
                if (row < m) {
                    const uint32_t col0 = n0 + c0;
                    if (EPI == AK_EPI_STORE_F32 || EPI == AK_EPI_ADD_F32) {
                        float* dst = reinterpret_cast<float*>(cptr) + (size_t)row * ldc + col0;
                        const bool vec = (col0 + 16 <= n) && ((ldc & 3u) == 0);
                        if (vec) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4) {
                                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                                if (EPI == AK_EPI_ADD_F32) {
                                    float4 o = *reinterpret_cast<float4*>(dst + j);
                                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                                }
                                *reinterpret_cast<float4*>(dst + j) = v;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (col0 + j < n) {
                                    float v = __uint_as_float(r[j]);
                                    if (EPI == AK_EPI_ADD_F32) v += dst[j];
                                    dst[j] = v;
                                }
                        }
                    } else {
                        bf16* dst = reinterpret_cast<bf16*>(cptr) + (size_t)row * ldc + col0;
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            v[j] = __uint_as_float(r[j]);
                            if (EPI == AK_EPI_SILU_BF16) v[j] = v[j] / (1.0f + __expf(-v[j]));
                        }
                        const bool vec = (col0 + 16 <= n) && ((ldc & 7u) == 0);
                        if (vec) {
                            uint32_t pk[8];
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                bf162 t = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                                pk[j] = *reinterpret_cast<uint32_t*>(&t);
                            }
                            *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            *reinterpret_cast<uint4*>(dst + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (col0 + j < n) dst[j] = __float2bfloat16_rn(v[j]);
                        }
                    }
                }
            }
        }
    }
    // ---------------- common exit
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && fail_flag) atomicExch(&g_gemm_status, fail_flag);
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int BN, int EPI>
static int launch_cfg(cudaStream_t st, const CUtensorMap& tmA, const CUtensorMap& tmB, void* c, uint32_t m, uint32_t n,
                      uint32_t k, uint32_t ldc) {
    using C = GemmCfg<BN>;
    static bool attr_set[64] = {};
    int dev = 0;
    AK_CUDA(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        AK_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        attr_set[dev & 63] = true;
    }
    dim3 grid(cdiv(n, BN), cdiv(m, GB_M));
    gemm_bf16_kernel<BN, EPI><<<grid, G_THREADS, C::SMEM_BYTES, st>>>(tmA, tmB, c, m, n, k, ldc);
    AK_COUNT_LAUNCH();
    AK_CHECK_LAUNCH();
    return AK_OK;
}

template <int BN>
static int launch_bn(cudaStream_t st, const void* a, const void* wt, void* c, uint32_t m, uint32_t n, uint32_t k,
                     uint32_t epi, uint32_t ldc) {
    CUtensorMap tmA, tmB;
    int rc = make_tmap_2d(&tmA, a, 2, k, m, (uint64_t)k * 2, GB_K, GB_M, TMA_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, wt, 2, k, n, (uint64_t)k * 2, GB_K, BN, TMA_SWIZZLE_128B);
    if (rc) return rc;
    switch (epi) {
        case AK_EPI_STORE_F32: return launch_cfg<BN, AK_EPI_STORE_F32>(st, tmA, tmB, c, m, n, k, ldc);
        case AK_EPI_ADD_F32: return launch_cfg<BN, AK_EPI_ADD_F32>(st, tmA, tmB, c, m, n, k, ldc);
        case AK_EPI_STORE_BF16: return launch_cfg<BN, AK_EPI_STORE_BF16>(st, tmA, tmB, c, m, n, k, ldc);
        case AK_EPI_SILU_BF16: return launch_cfg<BN, AK_EPI_SILU_BF16>(st, tmA, tmB, c, m, n, k, ldc);
    }
    set_error("gemm_bf16: unknown epilogue %u", epi);
    return AK_ERR_INVALID_ARG;
}

// Tile width: the narrowest N tile that still gives about one wave of CTAs keeps the weight
// stream spread over all SMs for small m (decode), wide tiles amortise the A tile for large m.
static uint32_t pick_bn(uint32_t m, uint32_t n) {
    const uint32_t mt = cdiv(m, GB_M);
    const uint32_t cands[5] = {256, 128, 64, 32, 16};
    for (int i = 0; i < 5; i++) {
        uint32_t bn = cands[i];
        if ((uint64_t)mt * cdiv(n, bn) >= 148) return bn;
    }
    return 16;
}

int launch_gemm_bf16(cudaStream_t st, const void* a, const void* wt, void* c, uint32_t m, uint32_t n, uint32_t k,
                     uint32_t epilogue, uint32_t ldc) {
    if (m == 0 || n == 0) return AK_OK;
    AK_REQUIRE(k >= 8 && k % 8 == 0, AK_ERR_UNSUPPORTED, "gemm_bf16: k (%u) must be a positive multiple of 8", k);
    AK_REQUIRE(((uintptr_t)a % 16) == 0 && ((uintptr_t)wt % 16) == 0 && ((uintptr_t)c % 16) == 0, AK_ERR_INVALID_ARG,
               "gemm_bf16: operands must be 16-byte aligned");
    if (ldc == 0) ldc = n;
    switch (pick_bn(m, n)) {
        case 256: return launch_bn<256>(st, a, wt, c, m, n, k, epilogue, ldc);
        case 128: return launch_bn<128>(st, a, wt, c, m, n, k, epilogue, ldc);
        case 64: return launch_bn<64>(st, a, wt, c, m, n, k, epilogue, ldc);
        case 32: return launch_bn<32>(st, a, wt, c, m, n, k, epilogue, ldc);
        default: return launch_bn<16>(st, a, wt, c, m, n, k, epilogue, ldc);
    }
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
    return launch_gemm_bf16(as_stream(stream), a, wt, c, m.m, m.n, m.k, epilogue, m.n);
}
