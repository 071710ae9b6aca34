// Host-side plumbing: thread-local error text, device/stream/memory helpers of the C ABI,
// and TMA tensor-map construction.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "kernels.h"
#include "tma.h"

namespace ak {

static thread_local char g_err[512] = "";
thread_local unsigned long long g_launch_count = 0;

bool pdl_enabled() {
    // AK_PDL=0 in the environment turns programmatic dependent launch off (for A/B timing)
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("AK_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

std::mutex& device_cache_mutex() {
    static std::mutex mu;
    return mu;
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    const char* base = strrchr(file, '/');
    set_error("CUDA error %d (%s) at %s:%d: %s", (int)e, cudaGetErrorString(e), base ? base + 1 : file, line, what);
    return (e == cudaErrorMemoryAllocation) ? AK_ERR_ALLOC : AK_ERR_CUDA;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, uint32_t elem_bytes, uint64_t cols, uint64_t rows,
                 uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows, TmaSwizzle swizzle) {
    EncodeTiledFn enc = get_encode();
    AK_REQUIRE(enc, AK_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available from this driver");
    AK_REQUIRE(((uintptr_t)base % 16) == 0 && (row_stride_bytes % 16) == 0, AK_ERR_INVALID_ARG,
               "tensor map: base and row pitch must be 16-byte aligned (base %p, pitch %llu)", base,
               (unsigned long long)row_stride_bytes);
    AK_REQUIRE(box_cols * elem_bytes % 16 == 0 && box_cols <= 256 && box_rows <= 256, AK_ERR_INVALID_ARG,
               "tensor map: bad box %u x %u", box_cols, box_rows);
    CUtensorMapDataType dt = (elem_bytes == 2) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapSwizzle sw = (swizzle == TMA_SWIZZLE_128B) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = enc(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    AK_REQUIRE(r == CUDA_SUCCESS, AK_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (cols %llu rows %llu pitch %llu box %ux%u)",
               (int)r, (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)row_stride_bytes, box_cols, box_rows);
    return AK_OK;
}

}  // namespace ak

using namespace ak;

extern "C" {

const char* ak_last_error_string(void) { return g_err; }
const char* ak_version(void) { return "akasha-b200 0.1 (sm_100a)"; }

int ak_device_count(int* out) {
    AK_REQUIRE(out, AK_ERR_INVALID_ARG, "ak_device_count: null pointer");
    AK_CUDA(cudaGetDeviceCount(out));
    return AK_OK;
}
int ak_set_device(int device) {
    AK_CUDA(cudaSetDevice(device));
    return AK_OK;
}
int ak_device_malloc(void** out, size_t bytes) {
    AK_REQUIRE(out, AK_ERR_INVALID_ARG, "ak_device_malloc: null pointer");
    AK_CUDA(cudaMalloc(out, bytes ? bytes : 16));
    return AK_OK;
}
int ak_device_free(void* p) {
    AK_CUDA(cudaFree(p));
    return AK_OK;
}
int ak_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
    AK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return AK_OK;
}
int ak_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
    AK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    AK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return AK_OK;
}
int ak_memset(void* dst, int value, size_t bytes, void* stream) {
    AK_CUDA(cudaMemsetAsync(dst, value, bytes, as_stream(stream)));
    return AK_OK;
}
int ak_stream_create(void** out) {
    AK_REQUIRE(out, AK_ERR_INVALID_ARG, "ak_stream_create: null pointer");
    cudaStream_t s;
    AK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out = s;
    return AK_OK;
}
int ak_stream_destroy(void* stream) {
    AK_CUDA(cudaStreamDestroy(as_stream(stream)));
    return AK_OK;
}
int ak_stream_synchronize(void* stream) {
    AK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return AK_OK;
}
int ak_host_alloc_pinned(void** out, size_t bytes) {
    AK_REQUIRE(out, AK_ERR_INVALID_ARG, "ak_host_alloc_pinned: null pointer");
    AK_CUDA(cudaMallocHost(out, bytes ? bytes : 16));
    return AK_OK;
}
int ak_host_free_pinned(void* p) {
    AK_CUDA(cudaFreeHost(p));
    return AK_OK;
}
unsigned long long ak_launch_count(void) { return g_launch_count; }

int ak_check_device_status(void* stream) {
    int rc = gemm_bf16_check_status(as_stream(stream));
    if (rc) return rc;
    unsigned int v = 0;
    rc = attn_decode_status(&v);
    if (rc) return rc;
    AK_REQUIRE(v == 0, AK_ERR_DEVICE_WAIT, "attn_decode_paged: a bounded device-side wait expired (code %u)", v);
    rc = prefill_tc_status(&v);
    if (rc) return rc;
    AK_REQUIRE(v == 0, AK_ERR_DEVICE_WAIT, "attn_prefill (tensor cores): a bounded device-side wait expired (code %u)", v);
    return AK_OK;
}

}  // extern "C"
