// Tensor-parallel exchange for models too large for one GPU's bandwidth budget (Llama-2-70B class).
//
// The reference runs a model on one device and has no multi-GPU path; this file has no counterpart there.  One
// process per GPU; each context joins a communicator of `size` ranks.  The decode path needs exactly one exchange
// per half-layer: the sum over ranks of the partial results of the row-parallel matrices (attention output and
// FFN down projections), `dim` floats each.  The exchange is NCCL's all-reduce on the context's stream (NVLink /
// NVSwitch underneath; capturable in the decode step's CUDA graph), so it orders itself between the GEMV that
// produces the partial and the one that consumes the sum.
//
// NCCL is resolved with dlopen when a communicator is first created: the single-GPU library has no link-time
// dependency on it and loads on machines without NCCL.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};
NcclApi g_nccl;

int load_nccl(slai_ctx* ctx) {
    if (g_nccl.ok) return SLAI_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        g_nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.lib) break;
    }
    if (!g_nccl.lib) return slai_set_error(ctx, SLAI_ERR_NCCL, "tp: cannot load libnccl.so.2 (%s)", dlerror());
#define SYM(field, name)                                                                      \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(g_nccl.lib, name));          \
    if (!g_nccl.field) return slai_set_error(ctx, SLAI_ERR_NCCL, "tp: libnccl lacks %s", name);
    SYM(GetUniqueId, "ncclGetUniqueId")
    SYM(CommInitRank, "ncclCommInitRank")
    SYM(CommDestroy, "ncclCommDestroy")
    SYM(AllReduce, "ncclAllReduce")
    SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
    g_nccl.ok = true;
    return SLAI_OK;
}

#define SLAI_CHECK_NCCL(ctx, expr)                                                                           \
    do {                                                                                                     \
        ncclResult_t _r = (expr);                                                                            \
        if (_r != ncclSuccess)                                                                               \
            return slai_set_error((ctx), SLAI_ERR_NCCL, "%s failed: %s", #expr, g_nccl.GetErrorString(_r)); \
    } while (0)

}  // namespace

static_assert(sizeof(ncclUniqueId) == SLAI_TP_ID_BYTES, "SLAI_TP_ID_BYTES must equal sizeof(ncclUniqueId)");

SLAI_API int slai_tp_unique_id(slai_ctx* ctx, void* h_id) {
    if (!ctx || !h_id) return SLAI_ERR_INVALID_ARG;
    int rc = load_nccl(ctx);
    if (rc) return rc;
    ncclUniqueId id;
    SLAI_CHECK_NCCL(ctx, g_nccl.GetUniqueId(&id));
    memcpy(h_id, &id, sizeof(id));
    return SLAI_OK;
}

SLAI_API int slai_tp_init(slai_ctx* ctx, const void* h_id, int rank, int size) {
    if (!ctx || !h_id) return SLAI_ERR_INVALID_ARG;
    SLAI_REQUIRE(ctx, size >= 1 && rank >= 0 && rank < size, SLAI_ERR_INVALID_ARG, "tp: rank %d of %d", rank, size);
    SLAI_REQUIRE(ctx, !ctx->tp_comm, SLAI_ERR_INVALID_ARG, "tp: this context already belongs to a group");
    int rc = load_nccl(ctx);
    if (rc) return rc;
    SLAI_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
    ncclUniqueId id;
    memcpy(&id, h_id, sizeof(id));
    ncclComm_t comm = nullptr;
    SLAI_CHECK_NCCL(ctx, g_nccl.CommInitRank(&comm, size, id, rank));
    ctx->tp_comm = comm;
    ctx->tp_rank = rank;
    ctx->tp_size = size;
    return SLAI_OK;
}

SLAI_API int slai_tp_shutdown(slai_ctx* ctx) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    if (ctx->tp_comm) {
        cudaStreamSynchronize(ctx->stream);
        g_nccl.CommDestroy(reinterpret_cast<ncclComm_t>(ctx->tp_comm));
        ctx->tp_comm = nullptr;
    }
    ctx->tp_rank = 0;
    ctx->tp_size = 1;
    return SLAI_OK;
}

int tp_all_reduce_sum(slai_ctx* ctx, const float* d_in, float* d_out, int64_t n) {
    SLAI_REQUIRE(ctx, ctx->tp_comm, SLAI_ERR_INVALID_ARG, "tp: the context has not joined a group (slai_tp_init)");
    SLAI_CHECK_NCCL(ctx, g_nccl.AllReduce(d_in, d_out, (size_t)n, ncclFloat, ncclSum, reinterpret_cast<ncclComm_t>(ctx->tp_comm), ctx->stream));
    return SLAI_OK;
}

SLAI_API int slai_tp_all_reduce_sum(slai_ctx* ctx, const float* d_in, float* d_out, int64_t n) {
    if (!ctx || !d_in || !d_out || n <= 0) return SLAI_ERR_INVALID_ARG;
    if (ctx->tp_size == 1) {
        if (d_in != d_out) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(d_out, d_in, (size_t)n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        return SLAI_OK;
    }
    return tp_all_reduce_sum(ctx, d_in, d_out, n);
}
