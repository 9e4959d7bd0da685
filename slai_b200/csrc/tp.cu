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
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
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
    SYM(AllGather, "ncclAllGather")
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
    SLAI_ENTER(ctx);
    int rc = load_nccl(ctx);
    if (rc) return rc;
    ncclUniqueId id;
    SLAI_CHECK_NCCL(ctx, g_nccl.GetUniqueId(&id));
    memcpy(h_id, &id, sizeof(id));
    return SLAI_OK;
}

SLAI_API int slai_tp_init(slai_ctx* ctx, const void* h_id, int rank, int size) {
    if (!ctx || !h_id) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
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

// ---- exchange over peer memory ---------------------------------------------------------------------------------
// NCCL's all-reduce costs a kernel launch and 10-20 us for the 32 KB this path exchanges.  With the ranks'
// exchange regions mapped into each other (CUDA IPC, NVLink peer access) the producing GEMV stores its partial
// rows straight into every rank's region -- each element as one 8-byte (value, sequence tag) store -- and the
// consuming GEMV sums the partials while it stages its input, polling the tags: no extra kernel, no flags or
// fences, one NVLink store latency.  Plain peer stores and local loads only; every wait is bounded.
namespace {
constexpr size_t XCHG_ELEMS = (size_t)2 * XCHG_MAX_RANKS * XCHG_MAX_DIM;
constexpr size_t XCHG_LOCAL_ELEMS = (size_t)2 * XCHG_MAX_DIM;  // two-level sums of this GPU
constexpr size_t XCHG_BYTES = (XCHG_ELEMS + XCHG_LOCAL_ELEMS) * sizeof(uint2) + 4096;  // the token counter lives in the last page

__global__ void tp_tick_kernel(unsigned int* tokseq) { *tokseq += 1; }
}  // namespace

static_assert(sizeof(cudaIpcMemHandle_t) == SLAI_TP_HANDLE_BYTES, "SLAI_TP_HANDLE_BYTES must equal sizeof(cudaIpcMemHandle_t)");

int tp_tick(slai_ctx* ctx) {
    tp_tick_kernel<<<1, 1, 0, ctx->stream>>>(ctx->xchg.d_tokseq);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}

SLAI_API int slai_tp_peer_export(slai_ctx* ctx, void* h_handle) {
    if (!ctx || !h_handle) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, ctx->tp_size >= 2 && ctx->tp_size <= XCHG_MAX_RANKS, SLAI_ERR_INVALID_ARG,
                 "tp: the peer exchange serves groups of 2..%d ranks (join one with slai_tp_init first)", XCHG_MAX_RANKS);
    SLAI_REQUIRE(ctx, !ctx->xchg_region, SLAI_ERR_INVALID_ARG, "tp: the exchange region is already exported");
    SLAI_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
    SLAI_CHECK_CUDA(ctx, cudaMalloc(&ctx->xchg_region, XCHG_BYTES));
    SLAI_CHECK_CUDA(ctx, cudaMemset(ctx->xchg_region, 0, XCHG_BYTES));
    SLAI_CHECK_CUDA(ctx, cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    SLAI_CHECK_CUDA(ctx, cudaIpcGetMemHandle(&h, ctx->xchg_region));
    memcpy(h_handle, &h, sizeof(h));
    return SLAI_OK;
}

SLAI_API int slai_tp_peer_attach(slai_ctx* ctx, const void* h_handles) {
    if (!ctx || !h_handles) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, ctx->xchg_region && !ctx->xchg_ready, SLAI_ERR_INVALID_ARG, "tp: export this rank's region first (once)");
    SLAI_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
    PeerExchange& X = ctx->xchg;
    X.ranks = ctx->tp_size;
    X.rank = ctx->tp_rank;
    for (int r = 0; r < X.ranks; r++) {
        void* base = ctx->xchg_region;
        if (r != X.rank) {
            cudaIpcMemHandle_t h;
            memcpy(&h, reinterpret_cast<const char*>(h_handles) + (size_t)r * sizeof(h), sizeof(h));
            cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return slai_set_error(ctx, SLAI_ERR_CUDA, "tp: cannot map rank %d's exchange region (%s); ranks must be separate processes "
                                      "on GPUs with peer access", r, cudaGetErrorString(e));
            }
        }
        X.slot_at[r] = reinterpret_cast<uint2*>(base);
    }
    X.local_sum = reinterpret_cast<uint2*>(ctx->xchg_region) + XCHG_ELEMS;
    X.d_tokseq = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(ctx->xchg_region) + (XCHG_ELEMS + XCHG_LOCAL_ELEMS) * sizeof(uint2));
    ctx->xchg_ready = true;
    return SLAI_OK;
}

// One process, one GPU: every rank's slot base is this context's own region, and the caller plays the ranks one after
// another by calling again with another `rank`.  Stores that would cross NVLink land in the same memory a peer
// would have written, so the exchange arithmetic (and its bounded waits) can be exercised without a second GPU.
SLAI_API int slai_tp_peer_loopback(slai_ctx* ctx, int ranks, int rank) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, ranks >= 2 && ranks <= XCHG_MAX_RANKS && rank >= 0 && rank < ranks, SLAI_ERR_INVALID_ARG,
                 "tp: loopback exchange of %d ranks, rank %d", ranks, rank);
    SLAI_REQUIRE(ctx, !ctx->tp_comm, SLAI_ERR_INVALID_ARG, "tp: this context belongs to a real group");
    if (!ctx->xchg_region) {
        SLAI_CHECK_CUDA(ctx, cudaMalloc(&ctx->xchg_region, XCHG_BYTES));
        SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(ctx->xchg_region, 0, XCHG_BYTES, ctx->stream));
    }
    PeerExchange& X = ctx->xchg;
    X.ranks = ranks;
    X.rank = rank;
    for (int r = 0; r < XCHG_MAX_RANKS; r++) X.slot_at[r] = r < ranks ? reinterpret_cast<uint2*>(ctx->xchg_region) : nullptr;
    X.local_sum = reinterpret_cast<uint2*>(ctx->xchg_region) + XCHG_ELEMS;
    X.d_tokseq = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(ctx->xchg_region) + (XCHG_ELEMS + XCHG_LOCAL_ELEMS) * sizeof(uint2));
    ctx->xchg_ready = false;  // models keep using NCCL / a real attachment; only the exchange operators below use the loopback
    ctx->xchg_loopback = true;
    return SLAI_OK;
}

SLAI_API int slai_tp_token_tick(slai_ctx* ctx) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, ctx->xchg_ready || ctx->xchg_loopback, SLAI_ERR_INVALID_ARG, "tp: no exchange region attached");
    return tp_tick(ctx);
}

static int exchange_check(slai_ctx* ctx, const slai_qmatrix* w, int index, int per_token) {
    SLAI_REQUIRE(ctx, ctx->xchg_ready || ctx->xchg_loopback, SLAI_ERR_INVALID_ARG, "tp: no exchange region attached");
    SLAI_REQUIRE(ctx, w->fmt != SLAI_FMT_F32, SLAI_ERR_UNSUPPORTED_FORMAT, "tp: the exchange operators take quantised matrices");
    SLAI_REQUIRE(ctx, per_token >= 1 && index >= 0 && index < per_token, SLAI_ERR_INVALID_ARG, "tp: exchange %d of %d per token", index, per_token);
    return SLAI_OK;
}

SLAI_API int slai_gemv_quant_partial(slai_ctx* ctx, const slai_qmatrix* w, const float* d_v, const float* d_resid, int index, int per_token) {
    if (!ctx || !w || !d_v) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    int rc = exchange_check(ctx, w, index, per_token);
    if (rc) return rc;
    GemvLaunch L;
    L.fmt = w->fmt; L.K = (int)w->ncols; L.nseg = 1;
    L.seg[0].w = w->data; L.seg[0].tile_bytes = w->tile_bytes; L.seg[0].rows = (int)w->nrows;
    L.v = d_v; L.out = nullptr; L.resid = d_resid; L.epi = EPI_XCHG;
    L.xchg = &ctx->xchg; L.xchg_out_idx1 = index + 1; L.xchg_per_token = per_token;
    SLAI_REQUIRE(ctx, d_resid || ctx->xchg.rank != 0, SLAI_ERR_INVALID_ARG, "tp: rank 0 adds the residual and needs d_resid");
    return gemv_launch(ctx, L);
}

SLAI_API int slai_gemv_quant_reduced(slai_ctx* ctx, float* d_out, const slai_qmatrix* w, const float* d_norm_w, float eps, int index,
                                     int per_token, float* d_sum_out) {
    if (!ctx || !w || !d_out || !d_norm_w || !d_sum_out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    int rc = exchange_check(ctx, w, index, per_token);
    if (rc) return rc;
    GemvLaunch L;
    L.fmt = w->fmt; L.K = (int)w->ncols; L.nseg = 1;
    L.seg[0].w = w->data; L.seg[0].tile_bytes = w->tile_bytes; L.seg[0].rows = (int)w->nrows;
    L.v = d_sum_out; L.out = d_out; L.pro = PRO_RMS; L.norm_w = d_norm_w; L.eps = eps; L.epi = EPI_STORE;
    L.xchg = &ctx->xchg; L.xchg_in_idx1 = index + 1; L.xchg_per_token = per_token; L.xsum_out = d_sum_out;
    return gemv_launch(ctx, L);
}

SLAI_API int slai_tp_shutdown(slai_ctx* ctx) {
    if (!ctx) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    if (ctx->xchg_region) {
        cudaStreamSynchronize(ctx->stream);
        if (ctx->xchg_ready)
            for (int r = 0; r < ctx->xchg.ranks; r++)
                if (r != ctx->xchg.rank && ctx->xchg.slot_at[r]) cudaIpcCloseMemHandle(ctx->xchg.slot_at[r]);
        cudaFree(ctx->xchg_region);
        ctx->xchg_region = nullptr;
        ctx->xchg_ready = false;
        ctx->xchg_loopback = false;
        ctx->xchg = PeerExchange{};
    }
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

// Every rank's `n` floats, concatenated in rank order, on every rank (the sharded logits: each rank computes the rows
// of the output matrix it holds).
int tp_all_gather(slai_ctx* ctx, const float* d_in, float* d_out, int64_t n) {
    SLAI_REQUIRE(ctx, ctx->tp_comm, SLAI_ERR_INVALID_ARG, "tp: the context has not joined a group (slai_tp_init)");
    SLAI_CHECK_NCCL(ctx, g_nccl.AllGather(d_in, d_out, (size_t)n, ncclFloat, reinterpret_cast<ncclComm_t>(ctx->tp_comm), ctx->stream));
    return SLAI_OK;
}

SLAI_API int slai_tp_all_reduce_sum(slai_ctx* ctx, const float* d_in, float* d_out, int64_t n) {
    if (!ctx || !d_in || !d_out || n <= 0) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    if (ctx->tp_size == 1) {
        if (d_in != d_out) SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(d_out, d_in, (size_t)n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        return SLAI_OK;
    }
    return tp_all_reduce_sum(ctx, d_in, d_out, n);
}
