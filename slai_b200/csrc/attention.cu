// Single-query attention over the KV cache (BatchedMultiqueryAttention::launch,
// crates/slai/src/ops/batched_multiquery_attention.rs:32-100; CPU twin :102-156).
//
// The reference issues four launches per layer (K^T q gemv, scale+mask, softmax, V att gemv) over an
// f32 cache and materialises the score matrix.  Here one kernel does the whole head: the positions
// 0..=pos are split over `n_splits` blocks per KV head (flash-decoding), each block computes scores for
// all query heads that share the KV head (GQA), a local softmax, and the weighted V sum; the last block
// to finish a KV head merges the splits with the usual (max, sum) rescaling in a fixed order.
// Cache element type is f16 or f32; strides are parameters so both the reference's position-major layout
// and the models' head-major layout are served.
#include "attention.cuh"

using namespace attn;

#ifndef SLAI_ATT_MINB
#define SLAI_ATT_MINB 4
#endif

namespace {

template <typename T, int MAXQ>
__global__ void __launch_bounds__(ATT_THREADS, SLAI_ATT_MINB) attn_kernel(const AttnParams P) {
    extern __shared__ __align__(16) unsigned char sm[];
#ifdef SLAI_TRACE
    unsigned long long tl0 = slai_globaltimer(), tl1 = 0;
#endif
    // The grid is sized for the longest context; the blocks of splits the current context does not use leave at once,
    // while the predecessor still runs, when the position is known not to be written by it.
    if (P.early && P.batch == 0 && (int)blockIdx.y >= attn_splits(P, __ldcg(P.d_pos) + 1)) return;
    prefetch_plan_issue(P.ahead, (int)(blockIdx.x + gridDim.x * blockIdx.y), (int)(gridDim.x * gridDim.y), (int)threadIdx.x, ATT_THREADS);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next kernel may start fetching its weights
#ifdef SLAI_TRACE
    tl1 = slai_globaltimer();
#endif
    if (P.batch > 0) {  // prompt processing: one query token per blockIdx.z
        const int b = (int)blockIdx.z;
        AttnParams Q = P;
        Q.q = P.q + (size_t)b * P.q_bs;
        Q.out = P.out + (size_t)b * P.out_bs;
        Q.part_o = P.part_o + (size_t)b * P.po_bs;
        Q.part_ml = P.part_ml + (size_t)b * P.pml_bs;
        Q.counters = P.counters + (size_t)b * gridDim.x;
        Q.kc = reinterpret_cast<const char*>(P.kc) + (size_t)b * P.cache_bs;
        Q.vc = reinterpret_cast<const char*>(P.vc) + (size_t)b * P.cache_bs;
        const int n = (P.seq_pos ? __ldcg(P.seq_pos + b) : P.pos0 + b) + 1;
        const int ns = n > 0 ? attn_splits(Q, n) : 0;  // a sequence left out of the step (negative position): nothing to do
        if ((int)blockIdx.y < ns) attn_item<T, MAXQ>(Q, blockIdx.x, blockIdx.y, ns, n, threadIdx.x, sm, 0);
    } else {
        const int n = __ldcg(P.d_pos) + 1;
        const int ns = attn_splits(P, n);
        if ((int)blockIdx.y < ns) attn_item<T, MAXQ>(P, blockIdx.x, blockIdx.y, ns, n, threadIdx.x, sm, 0);
    }
#ifdef SLAI_TRACE
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && P.tl) {
        unsigned long long st[TL_SLOTS] = {};
        st[0] = tl0;
        st[4] = tl1;
        st[13] = slai_globaltimer();
        slai_tl_append(P.tl, 999, st);
    }
#endif
}

template <typename T, int MAXQ>
int launch_t(slai_ctx* ctx, const AttnParams& P, int n_kv, size_t smem, bool pdl) {
    auto kern = attn_kernel<T, MAXQ>;
    static PerDeviceOnce attr;
    if (attr.need(ctx->device)) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        // Same shared-memory carve-out as the GEMV kernels it alternates with: no reconfiguration between launches.
        const char* co = getenv("SLAI_ATTN_CARVEOUT");
        if (!(co && co[0] == '0'))
            SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        attr.set(ctx->device);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_kv, P.n_splits, P.batch > 0 ? P.batch : 1);
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    SLAI_CHECK_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, P));
    return SLAI_OK;
}

}  // namespace

int ensure_scratch(slai_ctx* ctx, size_t bytes) {
    if (ctx->scratch_bytes >= bytes) return SLAI_OK;
    // Grow-only, and the outgrown buffer is kept until the context goes: a pass recorded earlier (slai_pass_*) still
    // launches kernels that point at it.  Growing at least doubles, so the retired buffers sum to less than the live one.
    if (bytes < 2 * ctx->scratch_bytes) bytes = 2 * ctx->scratch_bytes;
    void* fresh = nullptr;
    SLAI_CHECK_CUDA(ctx, cudaMalloc(&fresh, bytes));
    if (ctx->d_scratch) ctx->retired_scratch.push_back(ctx->d_scratch);
    ctx->d_scratch = fresh;
    ctx->scratch_bytes = bytes;
    return SLAI_OK;
}

static int pick_splits(int head_size, int esz, int n_max) {
    // One split per tile of positions, at most 64 (the kernel uses fewer while the context is short).
    const int tile = attn_tile_pos(head_size, esz);
    int n_splits = (n_max + tile - 1) / tile;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 64) n_splits = 64;
    return n_splits;
}

size_t attention_scratch_bytes(slai_ctx* ctx, int n_heads, int kv_mul, int head_size, int max_pos) {
    (void)ctx; (void)kv_mul;
    const int n_splits = pick_splits(head_size, 4, max_pos + 1);  // the f32 tile holds fewer positions: most splits
    const size_t po = (size_t)n_heads * n_splits * head_size * 4;
    const size_t pml = (size_t)n_heads * n_splits * 2 * 4;
    return ((po + 255) & ~(size_t)255) + pml + 256;
}

// Tile size, split count, copy width and shared memory of a launch.
static int attn_geometry(slai_ctx* ctx, AttnParams& P, int kv_dtype, int n_max, size_t* smem) {
    const int esz = kv_dtype == SLAI_KV_F16 ? 2 : 4;
    P.tile_pos = attn_tile_pos(P.hs, esz);
    P.n_splits = pick_splits(P.hs, esz, n_max);
    const uintptr_t bits = reinterpret_cast<uintptr_t>(P.kc) | reinterpret_cast<uintptr_t>(P.vc) | (uintptr_t)(P.pos_stride * esz) |
                           (uintptr_t)(P.head_stride * esz) | (uintptr_t)(P.hs * esz);
    SLAI_REQUIRE(ctx, (bits & 3) == 0, SLAI_ERR_INVALID_ARG, "attention: caches and strides must be 4-byte aligned");
    P.vec16 = (bits & 15) == 0;
    *smem = attn_item_bytes(P.kv_mul, P.hs, esz, P.tile_pos, P.n_splits);
    SLAI_REQUIRE(ctx, *smem <= 160 * 1024, SLAI_ERR_SHAPE, "attention: shared memory %zu too large", *smem);
    return SLAI_OK;
}

static int attention_launch_inner(slai_ctx* ctx, const AttnLaunch& A);
int attention_launch(slai_ctx* ctx, const AttnLaunch& A) {
    if (!ctx->stats_on) return attention_launch_inner(ctx, A);
    int rc = slai_stats_mark(ctx, STATS_OTHER);
    if (rc) return rc;
    if ((rc = attention_launch_inner(ctx, A))) return rc;
    return slai_stats_mark(ctx, STATS_ATTENTION);
}
static int attention_launch_inner(slai_ctx* ctx, const AttnLaunch& A) {
    SLAI_REQUIRE(ctx, A.kv_mul >= 1 && A.kv_mul <= 8 && A.n_heads % A.kv_mul == 0, SLAI_ERR_SHAPE,
                 "attention: kv_mul=%d must be in 1..8 and divide n_heads=%d", A.kv_mul, A.n_heads);
    SLAI_REQUIRE(ctx, A.head_size % 2 == 0 && A.head_size <= 64 * MAX_J, SLAI_ERR_SHAPE,
                 "attention: head_size=%d must be even and <= %d", A.head_size, 64 * MAX_J);
    const int share = attn_kv_share(A.kv_mul);
    const int n_kv = A.n_heads / A.kv_mul * share;  // virtual heads: the grid's x extent and the number of tickets
    const int kv_mul = A.kv_mul / share;
    SLAI_REQUIRE(ctx, n_kv <= 1024, SLAI_ERR_SHAPE, "attention: too many heads");
    const int n_max = A.max_pos + 1;
    AttnParams P;
    P.q = A.q; P.kc = A.kcache; P.vc = A.vcache;
    P.pos_stride = A.pos_stride; P.head_stride = A.head_stride;
    P.n_heads = A.n_heads; P.kv_mul = kv_mul; P.kv_share = share; P.hs = A.head_size;
    size_t smem = 0;
    {
        int rc = attn_geometry(ctx, P, A.kv_dtype, n_max, &smem);
        if (rc) return rc;
    }
    const size_t po = (size_t)A.n_heads * P.n_splits * A.head_size * 4;
    const size_t per_token = attention_scratch_bytes(ctx, A.n_heads, A.kv_mul, A.head_size, A.max_pos);
    const size_t need = per_token * (size_t)(A.batch > 0 ? A.batch : 1);
    SLAI_REQUIRE(ctx, A.batch == 0 || (A.scratch && A.batch_counters), SLAI_ERR_INVALID_ARG, "attention: a batch needs its own scratch and tickets");
    void* scratch = A.scratch;
    if (!scratch) {
        int rc = ensure_scratch(ctx, need);
        if (rc) return rc;
        scratch = ctx->d_scratch;
    } else {
        SLAI_REQUIRE(ctx, A.scratch_bytes >= need, SLAI_ERR_INVALID_ARG, "attention: scratch too small");
    }

    P.d_pos = A.d_pos;
    P.early = A.pos_stable ? 1 : 0;
    P.out = A.out;
    P.ahead = A.ahead;
#ifdef SLAI_TRACE
    P.tl = ctx->tl;
#endif
    P.part_o = reinterpret_cast<float*>(scratch);
    P.part_ml = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + ((po + 255) & ~(size_t)255));
    P.counters = A.batch > 0 ? A.batch_counters : ctx->d_counters + CNT_ATTN_TICKETS;
    P.batch = A.batch; P.pos0 = A.pos0; P.q_bs = A.q_batch_stride; P.out_bs = A.out_batch_stride;
    SLAI_REQUIRE(ctx, (A.cache_batch_stride == 0 && !A.d_pos_batch) || (A.batch > 0 && A.cache_batch_stride > 0 && A.d_pos_batch &&
                          A.cache_batch_stride % 4 == 0), SLAI_ERR_INVALID_ARG, "attention: a batch of sequences needs positions and a cache stride");
    P.cache_bs = A.cache_batch_stride; P.seq_pos = A.d_pos_batch;
    if (A.cache_batch_stride & 15) P.vec16 = 0;
    P.po_bs = (long long)(per_token / 4); P.pml_bs = (long long)(per_token / 4);  // every token's partials in its own slice of the scratch
    const bool f16 = A.kv_dtype == SLAI_KV_F16;
    if (kv_mul == 1) return f16 ? launch_t<__half, 1>(ctx, P, n_kv, smem, A.pdl) : launch_t<float, 1>(ctx, P, n_kv, smem, A.pdl);
    return f16 ? launch_t<__half, 2>(ctx, P, n_kv, smem, A.pdl) : launch_t<float, 2>(ctx, P, n_kv, smem, A.pdl);
}

int attention_tickets(int n_heads, int kv_mul) { return n_heads / kv_mul * attn_kv_share(kv_mul); }

// =================================================================================================
// Attention without any allocation (slai_attention_static).
//
// Some hosts hand every component its device memory once, up front, and then forbid further calls into the
// driver's allocator (a game or simulation engine embedding the model next to its own buffers, a serving
// process whose latency path must never reach cudaMalloc / cudaFree because both synchronise the device and can
// fail late).  `slai_attention` grows a per-context scratch buffer on demand, so such callers cannot use it.
// This variant keeps the flash-decoding partials, the per-head tickets and the position scalar in one
// file-scope device array of fixed size that every GPU loading the library holds until the process exits.
//
// The array's name is only a host-side handle: its device address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and the kernel is given that address.
// =================================================================================================
namespace {

constexpr size_t STATIC_PART_BYTES = SLAI_ATTENTION_STATIC_MAX_SCRATCH_BYTES;  // split partials
constexpr size_t STATIC_TICKET_BYTES = 4096;                                  // one ticket per KV head (<= 1024)
constexpr int STATIC_MAX_DEVICES = 64;

static __device__ __align__(256) unsigned char g_attn_static[STATIC_PART_BYTES + STATIC_TICKET_BYTES + 256];
static unsigned char* g_attn_static_ptr[STATIC_MAX_DEVICES];  // device address of the array, per device

__global__ void static_set_pos_kernel(int* dst, int pos) { *dst = pos; }

}  // namespace

SLAI_API int slai_attention_static(slai_ctx* ctx, const slai_attn_params* p, const float* d_q, const void* d_key_cache,
                                   const void* d_value_cache, int kv_dtype, float* d_xb) {
    if (!ctx || !p || !d_q || !d_key_cache || !d_value_cache || !d_xb) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, p->pos < p->seq_len, SLAI_ERR_SHAPE, "attention: pos=%u >= seq_len=%u", p->pos, p->seq_len);
    SLAI_REQUIRE(ctx, p->kv_mul >= 1 && p->kv_mul <= 8 && p->n_heads % p->kv_mul == 0 &&
                          p->kv_dim == p->n_heads / p->kv_mul * p->head_size,
                 SLAI_ERR_SHAPE, "attention: inconsistent head counts");
    SLAI_REQUIRE(ctx, p->head_size % 2 == 0 && p->head_size <= 64 * MAX_J, SLAI_ERR_SHAPE,
                 "attention: head_size=%u must be even and <= %d", p->head_size, 64 * MAX_J);
    SLAI_REQUIRE(ctx, kv_dtype == SLAI_KV_F16 || kv_dtype == SLAI_KV_F32, SLAI_ERR_INVALID_ARG, "attention: unknown cache type");
    const int n_heads = (int)p->n_heads, kv_mul = (int)p->kv_mul, hs = (int)p->head_size, pos = (int)p->pos;
    const int n_kv = n_heads / kv_mul;
    SLAI_REQUIRE(ctx, n_kv <= 1024, SLAI_ERR_SHAPE, "attention: too many KV heads");
    SLAI_REQUIRE(ctx, ctx->device >= 0 && ctx->device < STATIC_MAX_DEVICES, SLAI_ERR_INVALID_ARG, "attention: device index out of range");

    AttnParams P;
    P.q = d_q; P.kc = d_key_cache; P.vc = d_value_cache;
    P.pos_stride = p->kv_dim; P.head_stride = hs;
    P.n_heads = n_heads; P.kv_mul = kv_mul; P.hs = hs;
    size_t smem = 0;
    {
        int rc = attn_geometry(ctx, P, kv_dtype, pos + 1, &smem);
        if (rc) return rc;
    }
    const size_t po = (size_t)n_heads * P.n_splits * hs * 4;
    // Sized for the last position of this cache, not the current one: a shape that will not fit later in the
    // generation is refused at its first call.
    const size_t need = attention_scratch_bytes(ctx, n_heads, kv_mul, hs, (int)p->seq_len - 1);
    SLAI_REQUIRE(ctx, need <= STATIC_PART_BYTES, SLAI_ERR_SHAPE,
                 "slai_attention_static: this shape needs %zu bytes of split scratch at seq_len=%u, the built-in array holds %zu "
                 "(use slai_attention, which allocates)", need, p->seq_len, STATIC_PART_BYTES);

    // Set-up, once per device: resolve the array's device address with that device current (SLAI_ENTER made it so).
    if (!g_attn_static_ptr[ctx->device]) {
        void* sym = nullptr;
        SLAI_CHECK_CUDA(ctx, cudaGetSymbolAddress(&sym, g_attn_static));
        g_attn_static_ptr[ctx->device] = reinterpret_cast<unsigned char*>(sym);
    }
    unsigned char* base = g_attn_static_ptr[ctx->device];
    unsigned int* tickets = reinterpret_cast<unsigned int*>(base + STATIC_PART_BYTES);
    int* d_pos = reinterpret_cast<int*>(base + STATIC_PART_BYTES + STATIC_TICKET_BYTES);

    // The array keeps whatever the last call left: the tickets must start at zero, the position is rewritten.
    SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(tickets, 0, (size_t)n_kv * sizeof(unsigned int), ctx->stream));
    static_set_pos_kernel<<<1, 1, 0, ctx->stream>>>(d_pos, pos);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());

    P.d_pos = d_pos;
    P.out = d_xb;
    P.part_o = reinterpret_cast<float*>(base);
    P.part_ml = reinterpret_cast<float*>(base + ((po + 255) & ~(size_t)255));
    P.counters = tickets;
    const bool f16 = kv_dtype == SLAI_KV_F16;
    if (kv_mul == 1) return f16 ? launch_t<__half, 1>(ctx, P, n_kv, smem, false) : launch_t<float, 1>(ctx, P, n_kv, smem, false);
    if (kv_mul <= 4) return f16 ? launch_t<__half, 4>(ctx, P, n_kv, smem, false) : launch_t<float, 4>(ctx, P, n_kv, smem, false);
    return f16 ? launch_t<__half, 8>(ctx, P, n_kv, smem, false) : launch_t<float, 8>(ctx, P, n_kv, smem, false);
}
