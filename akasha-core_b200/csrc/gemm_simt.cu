// True-fp32 (FMA pipe) matmul family for the parity mode and the emitter-level ABI:
//   C[m,n] (+)= A[m,k] @ B[k,n], all row-major f32 (the reference's matmul / matmul_add,
//   src/nn/ops/emit.rs:19-126; arithmetic in wilupgu's MATMUL / MATMUL_ADD / GEMV / GEMV_ADD).
// m == 1 is the bandwidth-bound GEMV: the weight matrix is streamed exactly once with 128-bit
// loads, K is split over a thread-block CLUSTER and the partial sums are reduced through
// distributed shared memory in a fixed order (deterministic, no atomics).
#include <cooperative_groups.h>

#include "kernels.h"

namespace cg = cooperative_groups;

namespace ak {

// ------------------------------------------------------------------------------------ GEMV
constexpr int GEMV_WARPS = 8;
constexpr int GEMV_MAX_KS = 8;

template <int VEC>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, uint32_t n,
                uint32_t k, uint32_t flags) {
    pdl_wait();
    pdl_trigger();
    constexpr int CT = 32 * VEC;  // columns per CTA
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t ks = cluster.num_blocks();
    const uint32_t rank = cluster.block_rank();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.x * CT + lane * VEC;

    __shared__ float part[GEMV_WARPS][CT];
    __shared__ float cl_part[GEMV_MAX_KS][CT];  // rank 0 receives every rank's CTA partial here

    // K slice of this CTA
    uint32_t per = (k + ks - 1) / ks;
    uint32_t kb = rank * per;
    uint32_t ke = (kb + per < k) ? kb + per : k;
    if (kb > k) kb = k;

    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) acc[v] = 0.0f;

    const bool col_ok = (n0 + VEC - 1) < n;  // VEC divides n on the vector paths
    if (col_ok) {
        constexpr int UNROLL = 8;
        uint32_t kk = kb + warp;
        for (; kk + (UNROLL - 1) * GEMV_WARPS < ke; kk += UNROLL * GEMV_WARPS) {
            float xv[UNROLL];
            float wv[UNROLL][VEC];
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                uint32_t r = kk + u * GEMV_WARPS;
                xv[u] = __ldg(x + r);
                const float* p = w + (size_t)r * n + n0;
                if constexpr (VEC == 4) {
                    float4 t = __ldcs(reinterpret_cast<const float4*>(p));
                    wv[u][0] = t.x; wv[u][1] = t.y; wv[u][2] = t.z; wv[u][3] = t.w;
                } else if constexpr (VEC == 2) {
                    float2 t = __ldcs(reinterpret_cast<const float2*>(p));
                    wv[u][0] = t.x; wv[u][1] = t.y;
                } else {
                    wv[u][0] = __ldcs(p);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; u++)
#pragma unroll
                for (int v = 0; v < VEC; v++) acc[v] = fmaf(xv[u], wv[u][v], acc[v]);
        }
        for (; kk < ke; kk += GEMV_WARPS) {
            float xv = __ldg(x + kk);
            const float* p = w + (size_t)kk * n + n0;
#pragma unroll
            for (int v = 0; v < VEC; v++) acc[v] = fmaf(xv, p[v], acc[v]);
        }
    }
#pragma unroll
    for (int v = 0; v < VEC; v++) part[warp][lane * VEC + v] = acc[v];
    __syncthreads();

    // CTA partial (fixed warp order), sent to rank 0's shared memory
    float cta_sum = 0.0f;
    if (threadIdx.x < CT) {
#pragma unroll
        for (int i = 0; i < GEMV_WARPS; i++) cta_sum += part[i][threadIdx.x];
        float* dst = cluster.map_shared_rank(&cl_part[0][0], 0);
        dst[rank * CT + threadIdx.x] = cta_sum;
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x < CT) {
        uint32_t col = blockIdx.x * CT + threadIdx.x;
        if (col < n) {
            float s = 0.0f;
            for (uint32_t r = 0; r < ks; r++) s += cl_part[r][threadIdx.x];
            if (flags & GEMM_SILU) s = s / (1.0f + expf(-s));
            if (flags & GEMM_ADD) s = y[col] + s;
            y[col] = s;
        }
    }
}

static uint32_t pow2_floor(uint32_t v) {
    uint32_t p = 1;
    while (p * 2 <= v) p *= 2;
    return p;
}

template <int VEC>
static int gemv_launch(cudaStream_t st, const float* x, const float* w, float* y, uint32_t n, uint32_t k, uint32_t flags) {
    constexpr int CT = 32 * VEC;
    uint32_t col_tiles = cdiv(n, CT);
    uint32_t ks = 1;
    if (col_tiles < 296) ks = pow2_floor(296 / col_tiles);
    if (ks > GEMV_MAX_KS) ks = GEMV_MAX_KS;
    while (ks > 1 && k / ks < 2 * GEMV_WARPS) ks /= 2;
    return launch_k(gemv_f32_kernel<VEC>, dim3(col_tiles, ks, 1), dim3(GEMV_WARPS * 32), 0, st, dim3(1, ks, 1), x, w, y, n, k, flags);
}

static int launch_gemv_f32(cudaStream_t st, const float* x, const float* w, float* y, uint32_t n, uint32_t k, uint32_t flags) {
    bool a16 = ((uintptr_t)w % 16) == 0, a8 = ((uintptr_t)w % 8) == 0;
    // wide loads when the matrix is large enough to fill the machine with 128-column tiles
    if ((n % 4) == 0 && a16 && n >= 4096) return gemv_launch<4>(st, x, w, y, n, k, flags);
    if ((n % 2) == 0 && a8 && n >= 1024) return gemv_launch<2>(st, x, w, y, n, k, flags);
    return gemv_launch<1>(st, x, w, y, n, k, flags);
}

// ------------------------------------------------------------------------------------ GEMM
// 64x64 tile, BK = 16, 256 threads, 4x4 accumulators per thread, k ascending.
constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c, uint32_t m, uint32_t n,
                uint32_t k, uint32_t flags) {
    pdl_wait();
    pdl_trigger();
    __shared__ float As[BK][BM + 4];  // transposed A tile
    __shared__ float Bs[BK][BN + 4];
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < k; k0 += BK) {
        // A tile: 64 rows x 16 k -> 1024 elements, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t e = threadIdx.x + i * 256;
            uint32_t r = e >> 4, kk = e & 15;
            uint32_t gr = m0 + r, gk = k0 + kk;
            As[kk][r] = (gr < m && gk < k) ? a[(size_t)gr * k + gk] : 0.0f;
        }
        // B tile: 16 k x 64 cols
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t e = threadIdx.x + i * 256;
            uint32_t kk = e >> 6, cc = e & 63;
            uint32_t gk = k0 + kk, gc = n0 + cc;
            Bs[kk][cc] = (gk < k && gc < n) ? b[(size_t)gk * n + gc] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            float ar[4] = {av.x, av.y, av.z, av.w};
            float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t r = m0 + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t col = n0 + tx * 4 + j;
            if (col >= n) continue;
            float s = acc[i][j];
            if (flags & GEMM_SILU) s = s / (1.0f + expf(-s));
            float* p = c + (size_t)r * n + col;
            if (flags & GEMM_ADD) s = *p + s;
            *p = s;
        }
    }
}

int launch_gemm_f32(cudaStream_t st, const float* a, const float* b, float* c, uint32_t m, uint32_t n, uint32_t k,
                    uint32_t flags) {
    if (m == 0 || n == 0) return AK_OK;
    if (m == 1 && k > 0) return launch_gemv_f32(st, a, b, c, n, k, flags);
    dim3 grid(cdiv(n, BN), cdiv(m, BM));
    AK_TRY(launch_k(gemm_f32_kernel, dim3(grid), dim3(256), 0, st, NO_CLUSTER, a, b, c, m, n, k, flags));
    return AK_OK;
}

}  // namespace ak

using namespace ak;
extern "C" {
int ak_matmul(void* stream, const float* a, const float* b, float* c, ak_matmul_meta m) {
    AK_REQUIRE(a && b && c, AK_ERR_INVALID_ARG, "ak_matmul: null pointer");
    return launch_gemm_f32(as_stream(stream), a, b, c, m.m, m.n, m.k, 0);
}
int ak_matmul_add(void* stream, const float* a, const float* b, float* c, ak_matmul_meta m) {
    AK_REQUIRE(a && b && c, AK_ERR_INVALID_ARG, "ak_matmul_add: null pointer");
    return launch_gemm_f32(as_stream(stream), a, b, c, m.m, m.n, m.k, GEMM_ADD);
}
}
