// The exchange steps of the sharded mixture-of-experts configuration: one process per GPU, NCCL over NVLink.
//
// Two sums cross the GPUs per routed layer, both f32 all-reduces on the session's stream:
//   - attention is tensor-parallel over heads, so every rank's o_proj yields the partial sums of its own head
//     columns ([rows, d_model]); their sum is the full projection;
//   - experts are sharded, so every rank computes the (row, slot) outputs of its own experts and leaves zeros for
//     the others ([rows * k, d_model]); adding zeros is exact, so after the sum every rank holds the same per-slot
//     values a single GPU computes, and the slot-ordered weighted sum that follows is bit-identical on every rank.
// NCCL is loaded at run time (the library the process already uses, e.g. the one torch.distributed loaded), so
// libtsb itself has no link-time dependency on it.  The few prototypes used are NCCL's public C API.
#include <dlfcn.h>

#include "common.cuh"

namespace {

struct NcclUniqueId {
    char internal[128];
};
using NcclComm = void*;
constexpr int kNcclFloat32 = 7, kNcclSum = 0;

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    std::string error;
};

NcclApi& nccl() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    const char* env = getenv("TSB_NCCL_LIB");
    const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        if (!n || !*n) continue;
        api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) break;
    }
    if (!api.handle) {
        api.error = "libnccl.so.2 could not be loaded (set TSB_NCCL_LIB to its path)";
        return api;
    }
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(api.handle, "ncclAllReduce"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce) {
        api.error = "the loaded NCCL library lacks one of ncclGetUniqueId / ncclCommInitRank / ncclCommDestroy / ncclAllReduce";
        api.handle = nullptr;
    }
    return api;
}

}  // namespace

struct tsb_comm {
    tsb_ctx* ctx = nullptr;
    NcclComm comm = nullptr;
    int rank = 0, world = 1;
};

cudaError_t comm_all_reduce_f32(tsb_comm* c, cudaStream_t st, float* buf, size_t count) {
    if (!c || c->world <= 1 || count == 0) return cudaSuccess;
    NcclApi& api = nccl();
    if (!api.handle || !c->comm) return cudaErrorNotReady;
    const int rc = api.AllReduce(buf, buf, count, kNcclFloat32, kNcclSum, c->comm, st);
    if (rc != 0) {
        c->ctx->last_error = std::string("ncclAllReduce failed: ") + (api.GetErrorString ? api.GetErrorString(rc) : "?");
        return cudaErrorUnknown;
    }
    c->ctx->launches++;
    return cudaSuccess;
}
int comm_world(const tsb_comm* c) { return c ? c->world : 1; }
int comm_rank(const tsb_comm* c) { return c ? c->rank : 0; }

extern "C" {

int32_t tsb_comm_unique_id(tsb_ctx* ctx, void* out_128_bytes) {
    if (!ctx || !out_128_bytes) return TSB_ERR_INVALID;
    NcclApi& api = nccl();
    if (!api.handle) return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "%s", api.error.c_str());
    NcclUniqueId id;
    const int rc = api.GetUniqueId(&id);
    if (rc != 0) return tsb_fail(ctx, TSB_ERR_CUDA, "ncclGetUniqueId failed: %s", api.GetErrorString ? api.GetErrorString(rc) : "?");
    memcpy(out_128_bytes, id.internal, sizeof id.internal);
    return TSB_OK;
}

int32_t tsb_comm_create(tsb_ctx* ctx, const void* unique_id_128_bytes, int32_t rank, int32_t world, tsb_comm** out) {
    if (!ctx || !out) return TSB_ERR_INVALID;
    *out = nullptr;
    TSB_REQUIRE(ctx, world >= 1 && rank >= 0 && rank < world, "rank %d outside a world of %d", rank, world);
    tsb_comm* c = new (std::nothrow) tsb_comm();
    if (!c) return TSB_ERR_OOM;
    c->ctx = ctx, c->rank = rank, c->world = world;
    if (world > 1) {
        TSB_REQUIRE(ctx, unique_id_128_bytes, "a world of more than one rank needs the unique id of rank 0");
        NcclApi& api = nccl();
        if (!api.handle) {
            delete c;
            return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "%s", api.error.c_str());
        }
        DeviceGuard g(ctx);
        NcclUniqueId id;
        memcpy(id.internal, unique_id_128_bytes, sizeof id.internal);
        const int rc = api.CommInitRank(&c->comm, world, id, rank);
        if (rc != 0) {
            delete c;
            return tsb_fail(ctx, TSB_ERR_CUDA, "ncclCommInitRank failed: %s", api.GetErrorString ? api.GetErrorString(rc) : "?");
        }
    }
    *out = c;
    return TSB_OK;
}

void tsb_comm_destroy(tsb_comm* c) {
    if (!c) return;
    if (c->comm) {
        DeviceGuard g(c->ctx);
        cudaDeviceSynchronize();
        nccl().CommDestroy(c->comm);
    }
    delete c;
}

int32_t tsb_comm_all_reduce_f32(tsb_comm* c, tsb_stream s, void* buf_f32_dev, size_t count) {
    if (!c) return TSB_ERR_INVALID;
    TSB_REQUIRE(c->ctx, buf_f32_dev || count == 0, "null buffer");
    DeviceGuard g(c->ctx);
    if (comm_all_reduce_f32(c, (cudaStream_t)s, static_cast<float*>(buf_f32_dev), count) != cudaSuccess)
        return tsb_fail(c->ctx, TSB_ERR_CUDA, "all-reduce failed: %s", c->ctx->last_error.c_str());
    return TSB_OK;
}

}  // extern "C"
