// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry point, so the library needs no link-time dependency on libcuda) and the
// device-side tiled load.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace ak {

enum TmaSwizzle { TMA_SWIZZLE_NONE = 0, TMA_SWIZZLE_128B = 3 };

// 2-D row-major tensor [rows, cols] of `elem_bytes`-byte elements (2 = bf16, 4 = f32), row pitch
// `row_stride_bytes` (multiple of 16). Box = [box_rows, box_cols]; out-of-range elements read 0.
int make_tmap_2d(CUtensorMap* out, const void* base, uint32_t elem_bytes, uint64_t cols, uint64_t rows,
                 uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows, TmaSwizzle swizzle);

#ifdef __CUDACC__
// Tiled 2-D load, completion counted in bytes on `bar`. x (the innermost coordinate) times the
// element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
#endif

}  // namespace ak
