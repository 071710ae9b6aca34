// Tensor-parallel plumbing: NCCL all-reduce after the row-split projections (out-proj, ffn-down)
// of the 2-way tensor-parallel variant. NCCL is loaded with dlopen at first use, so the library
// itself has no link-time dependency on it (single-GPU hosts never touch it).
// The reference has no parallelism of any kind (single device, src/main.rs:366); this is new.
#include <dlfcn.h>
#include <string.h>

#include "model.h"

namespace ak {

typedef struct { char internal[128]; } NcclUniqueId;
typedef int (*nccl_get_unique_id_t)(NcclUniqueId*);
typedef int (*nccl_comm_init_rank_t)(void** comm, int nranks, NcclUniqueId id, int rank);
typedef int (*nccl_comm_destroy_t)(void* comm);
typedef int (*nccl_all_reduce_t)(const void* send, void* recv, size_t count, int dtype, int op, void* comm, cudaStream_t st);
typedef const char* (*nccl_get_error_string_t)(int);

struct NcclApi {
    void* handle = nullptr;
    nccl_get_unique_id_t get_unique_id = nullptr;
    nccl_comm_init_rank_t comm_init_rank = nullptr;
    nccl_comm_destroy_t comm_destroy = nullptr;
    nccl_all_reduce_t all_reduce = nullptr;
    nccl_get_error_string_t get_error_string = nullptr;
};

static NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (api.handle) {
            api.get_unique_id = (nccl_get_unique_id_t)dlsym(api.handle, "ncclGetUniqueId");
            api.comm_init_rank = (nccl_comm_init_rank_t)dlsym(api.handle, "ncclCommInitRank");
            api.comm_destroy = (nccl_comm_destroy_t)dlsym(api.handle, "ncclCommDestroy");
            api.all_reduce = (nccl_all_reduce_t)dlsym(api.handle, "ncclAllReduce");
            api.get_error_string = (nccl_get_error_string_t)dlsym(api.handle, "ncclGetErrorString");
        }
    }
    if (!api.handle || !api.get_unique_id || !api.comm_init_rank || !api.all_reduce) return nullptr;
    return &api;
}

static int nccl_fail(NcclApi* a, int rc, const char* what) {
    set_error("NCCL error %d (%s) in %s", rc, a->get_error_string ? a->get_error_string(rc) : "?", what);
    return AK_ERR_CUDA;
}

// ncclFloat32 = 7, ncclSum = 0 (nccl.h enums, stable across NCCL 2.x)
int tp_all_reduce_f32(ak_ctx* ctx, float* buf, size_t count) {
    if (!ctx->tp_comm || ctx->tp_size <= 1) return AK_OK;
    NcclApi* a = nccl_api();
    AK_REQUIRE(a, AK_ERR_UNSUPPORTED, "NCCL is not available");
    int rc = a->all_reduce(buf, buf, count, 7, 0, ctx->tp_comm, ctx->stream);
    if (rc != 0) return nccl_fail(a, rc, "ncclAllReduce");
    return AK_OK;
}

}  // namespace ak

using namespace ak;

extern "C" {

int ak_tp_unique_id(void* out128) {
    AK_REQUIRE(out128, AK_ERR_INVALID_ARG, "ak_tp_unique_id: null pointer");
    NcclApi* a = nccl_api();
    AK_REQUIRE(a, AK_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded");
    NcclUniqueId id;
    int rc = a->get_unique_id(&id);
    if (rc != 0) return nccl_fail(a, rc, "ncclGetUniqueId");
    memcpy(out128, &id, sizeof(id));
    return AK_OK;
}

int ak_ctx_tp_init(ak_ctx* ctx, uint32_t tp_size, uint32_t tp_rank, const void* unique_id128) {
    AK_REQUIRE(ctx && unique_id128, AK_ERR_INVALID_ARG, "ak_ctx_tp_init: null pointer");
    AK_REQUIRE(tp_size >= 1 && tp_size <= 8 && tp_rank < tp_size, AK_ERR_INVALID_ARG, "ak_ctx_tp_init: bad tp_size/tp_rank");
    AK_REQUIRE(!ctx->tp_comm, AK_ERR_INVALID_ARG, "ak_ctx_tp_init: already initialised");
    ctx->tp_size = tp_size;
    ctx->tp_rank = tp_rank;
    if (tp_size == 1) return AK_OK;
    NcclApi* a = nccl_api();
    AK_REQUIRE(a, AK_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded");
    AK_CUDA(cudaSetDevice(ctx->device));
    NcclUniqueId id;
    memcpy(&id, unique_id128, sizeof(id));
    int rc = a->comm_init_rank(&ctx->tp_comm, (int)tp_size, id, (int)tp_rank);
    if (rc != 0) return nccl_fail(a, rc, "ncclCommInitRank");
    return AK_OK;
}

int ak_ctx_tp_shutdown(ak_ctx* ctx) {
    if (!ctx || !ctx->tp_comm) return AK_OK;
    NcclApi* a = nccl_api();
    if (a && a->comm_destroy) a->comm_destroy(ctx->tp_comm);
    ctx->tp_comm = nullptr;
    return AK_OK;
}

}  // extern "C"
