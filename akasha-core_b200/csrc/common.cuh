// Shared helpers for the sm_100a kernels: error plumbing, dtype traits, PTX wrappers for
// mbarrier / bulk-async (TMA) copies with BOUNDED waits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/akasha_b200.h"

namespace ak {

// This library is written for one part: B200, 148 SMs (two dies of 74). Grid sizing and launch plans use the figure.
constexpr uint32_t B200_SMS = 148;

// ---- host-side error plumbing -------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define AK_CUDA(call)                                                            \
    do {                                                                         \
        cudaError_t _e = (call);                                                 \
        if (_e != cudaSuccess) return ak::cuda_fail(_e, #call, __FILE__, __LINE__); \
    } while (0)

#define AK_CHECK_LAUNCH() AK_CUDA(cudaGetLastError())

#define AK_TRY(expr)              \
    do {                          \
        int _rc = (expr);         \
        if (_rc) return _rc;      \
    } while (0)

#define AK_REQUIRE(cond, code, ...)    \
    do {                               \
        if (!(cond)) {                 \
            ak::set_error(__VA_ARGS__); \
            return (code);             \
        }                              \
    } while (0)

static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
static inline unsigned cdiv(unsigned a, unsigned b) { return (a + b - 1) / b; }
static inline size_t cdiv64(size_t a, size_t b) { return (a + b - 1) / b; }

// Programmatic dependent launch (PDL): kernels of the per-step chain are launched with the
// programmatic-stream-serialization attribute, call pdl_wait() before touching global memory
// (it returns once every prerequisite grid has completed and flushed) and pdl_trigger() right
// after, which lets the NEXT kernel's blocks be scheduled early and run their prologue while this
// grid drains. Without the launch attribute both instructions are no-ops.
bool pdl_enabled();

// One mutex for the small per-device caches kept in function-local statics (kernel attributes already set,
// symbol addresses already looked up): the library may be driven from one host thread per GPU.
std::mutex& device_cache_mutex();

// Number of kernel launches issued by this library on the calling thread (for the benchmark's
// `gpu_launches` claim).
extern thread_local unsigned long long g_launch_count;
#define AK_COUNT_LAUNCH() (++ak::g_launch_count)

// ---- device helpers ------------------------------------------------------------------------
#ifdef __CUDACC__

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

template <typename T> struct Cvt;
template <> struct Cvt<float> {
    __device__ static __forceinline__ float to_f(float v) { return v; }
    __device__ static __forceinline__ float from_f(float v) { return v; }
};
template <> struct Cvt<bf16> {
    __device__ static __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ bf16 from_f(float v) { return __float2bfloat16_rn(v); }
};

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// RoPE rotation of one adjacent pair (src/shaders/cpu.rs:101-106): one rounding per operation (no fused
// multiply-add), so that every kernel that rotates a pair -- the split + append kernel, the decode attention that
// rotates its own query and new key -- produces the same bits, the bits of the reference's CPU arithmetic.
__device__ __forceinline__ void rope_rotate(float x0, float x1, float cs, float sn, float& o0, float& o1) {
    o0 = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
    o1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after roughly a second and returns false. The caller records an error
// in its status word and unwinds; it never spins forever.
#ifndef AK_WAIT_FAST_POLLS
#define AK_WAIT_FAST_POLLS 4096u
#endif
#ifndef AK_WAIT_SLOW_POLLS
#define AK_WAIT_SLOW_POLLS 2000000u
#endif
#ifndef AK_WAIT_MAX_CYCLES
#define AK_WAIT_MAX_CYCLES (1ll << 31)  // about a second of SM clock
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < AK_WAIT_FAST_POLLS; i++)
        if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 0; i < AK_WAIT_SLOW_POLLS; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > AK_WAIT_MAX_CYCLES) return false;
        __nanosleep(128);
    }
    return false;
}

// ---- bulk async copy (TMA, untiled): global -> shared, completion on an mbarrier ------------
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Launch helper for the per-step chain: optional thread-block cluster, PDL attribute when enabled.
template <typename... KArgs, typename... Args>
static inline int launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, dim3 cluster,
                           Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned na = 0;
    if (cluster.x * cluster.y * cluster.z > 0) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = cluster.x;
        attr[na].val.clusterDim.y = cluster.y;
        attr[na].val.clusterDim.z = cluster.z;
        na++;
    }
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<Args&&>(args)...);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx", __FILE__, __LINE__);
    AK_COUNT_LAUNCH();
    return AK_OK;
}
static const dim3 NO_CLUSTER(0, 0, 0);

#endif  // __CUDACC__

}  // namespace ak
