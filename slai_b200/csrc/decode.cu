// All layers of one decoded token in ONE persistent kernel (Llama2::launch's layer loop,
// crates/slai/src/models/llama2/transformer.rs:325-366).
//
// Launching the five kernels of a layer separately costs more than the work they do at batch 1: each launch
// pays kernel start-up, a cold ring, and a drain before the next one may start.  Here 148 blocks of threads (one
// per SM, cooperative launch) stay resident for the whole token and walk the phases
//     norm+QKV+RoPE+KV-append | attention | O+residual | norm+gate/up+SiLU | down+residual
// of every layer, separated by grid-wide barriers (one atomic arrive + bounded spin per block of threads).  The
// weight ring of gemv_kernel.cuh is driven by a program that lists every GEMV of every layer, so while a block
// waits at a barrier or runs the attention phase its ring already holds the first blocks of the next GEMV.
// Activations written in one phase and read in the next travel through L2 (ld.global.cg); nothing is read
// through L1 that another SM may have written during the launch.
#include "gemv_kernel.cuh"
#include "attention.cuh"

using namespace gemvk;
using attn::AttnParams;


namespace {

// The program of the ring producer: entry 4*l + k is GEMV k (QKV, O, gate/up, down) of layer l.  Everything comes
// from the kernel's parameter block.
struct LayerProg {
    const DecodeParams& D;
    __device__ __forceinline__ int size() const { return 4 * D.n_layers; }
    __device__ __forceinline__ ProgGeom geom(int idx) const {
        const int k = idx & 3;
        ProgGeom g;
        g.nsteps = k == 3 ? D.nsteps_hidden : D.nsteps_dim;
        g.nmat = k == 2 ? 2 : 1;
        g.items_base = D.items_base[k];
        g.items_rem = D.items_rem[k];
        return g;
    }
    __device__ __forceinline__ const uint8_t* tile_ptr(int idx, int item, int mat) const {
        const DecodeLayerPtrs& W = D.layer[idx >> 2];
        const int k = idx & 3;
        if (k == 0) {
            const int t1 = D.dim >> 4, t2 = (D.dim + D.kv_dim) >> 4;
            const uint8_t* w = W.wq;
            int t = item;
            if (item >= t1) { w = W.wk; t = item - t1; }
            if (item >= t2) { w = W.wv; t = item - t2; }
            return w + (size_t)t * D.tile_bytes_dim;
        }
        if (k == 1) return W.wo + (size_t)item * D.tile_bytes_dim;
        if (k == 2) return (mat ? W.wup : W.wgate) + (size_t)item * D.tile_bytes_dim;
        return W.wdown + (size_t)item * D.tile_bytes_hidden;
    }
};

// Parameters of GEMV phase k (0 QKV, 1 O, 2 gate/up, 3 down) of layer l, assembled in registers from the
// parameter block.
__device__ __forceinline__ GemvParams phase_params(const DecodeParams& D, int l, int k) {
    const DecodeLayerPtrs& W = D.layer[l];
    const bool qkv = k == 0, op = k == 1, gu = k == 2, dn = k == 3;
    GemvParams P{};
    P.nstage = D.nstage;
    P.step_bytes = D.step_bytes;
    P.stage_stride = D.stage_stride;
    P.dig_region = D.dig_region;
    P.err_flag = D.err_flag;
    P.wait_limit = D.wait_limit;
    P.eps = D.eps;
    P.nseg = qkv ? 3 : gu ? 2 : 1;
    P.nmat = gu ? 2 : 1;
    P.K = dn ? D.hidden : D.dim;
    P.nsteps = dn ? D.nsteps_hidden : D.nsteps_dim;
    P.n_items = qkv ? (D.dim + 2 * D.kv_dim) >> 4 : gu ? D.hidden >> 4 : D.dim >> 4;
    P.items_base = D.items_base[k];
    P.items_rem = D.items_rem[k];
    P.seg[0].w = qkv ? W.wq : op ? W.wo : gu ? W.wgate : W.wdown;
    P.seg[0].tile_bytes = dn ? D.tile_bytes_hidden : D.tile_bytes_dim;
    P.seg[0].rows = gu ? D.hidden : D.dim;
    P.seg[0].bias = qkv ? W.bq : nullptr;
    P.seg[1].w = qkv ? W.wk : W.wup;
    P.seg[1].tile_bytes = D.tile_bytes_dim;
    P.seg[1].rows = qkv ? D.kv_dim : D.hidden;
    P.seg[1].tile0 = D.dim >> 4;
    P.seg[1].bias = qkv ? W.bk : nullptr;
    P.seg[1].role = 1;
    P.seg[2].w = W.wv;
    P.seg[2].tile_bytes = D.tile_bytes_dim;
    P.seg[2].rows = D.kv_dim;
    P.seg[2].tile0 = (D.dim + D.kv_dim) >> 4;
    P.seg[2].bias = W.bv;
    P.seg[2].role = 2;
    P.v = (qkv || gu) ? D.x : op ? D.xb : D.hb;
    P.out = qkv ? D.q : gu ? D.hb : D.x;
    P.resid = D.x;
    P.norm_w = qkv ? W.attn_norm : W.ffn_norm;
    P.rope = 1; P.rope_theta = D.rope_theta; P.rope_cs = nullptr; P.head_size = D.head_size; P.d_pos = D.d_pos;
    P.kcache = W.kcache; P.vcache = W.vcache; P.k_out = nullptr; P.kv_f16 = D.kv_f16;
    P.kv_pos_stride = D.head_size; P.kv_head_stride = (long long)D.seq_len * D.head_size;
#ifdef SLAI_TRACE
    P.trace = nullptr;
    P.tl = nullptr;
#endif
    return P;
}

__device__ __forceinline__ AttnParams attn_params(const DecodeParams& D, int l) {
    const DecodeLayerPtrs& W = D.layer[l];
    AttnParams A;
    A.q = D.q; A.kc = W.kcache; A.vc = W.vcache;
    A.pos_stride = D.head_size; A.head_stride = (long long)D.seq_len * D.head_size;
    A.n_heads = D.n_heads; A.kv_mul = D.kv_mul; A.hs = D.head_size;
    A.d_pos = D.d_pos; A.n_splits = D.n_splits; A.tile_pos = D.tile_pos; A.vec16 = D.vec16;
    A.out = D.xb; A.part_o = D.part_o; A.part_ml = D.part_ml;
    A.counters = D.counters;
    return A;
}

// Grid-wide barrier: every block of threads arrives once per epoch; bounded spin (error flag 2 on expiry).
__device__ __forceinline__ void grid_sync(const DecodeParams& D, unsigned int& epoch) {
    __syncthreads();
    if (threadIdx.x == 0) {
        epoch++;
        __threadfence();
        atomicAdd(D.bar, 1u);
        const unsigned int target = epoch * gridDim.x;
        for (int it = 0;; it++) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(D.bar) : "memory");
            if (v >= target) break;
            if ((unsigned int)it > 4u * D.wait_limit) {
                atomicExch(D.err_flag, 2u);
                break;
            }
            if (it > 64) __nanosleep(32);
        }
        __threadfence();
    }
    __syncthreads();
}

// Attention phase: four items (KV head, split) at a time per block of threads, 128 threads each.
template <typename KV, int MAXQ>
__device__ __forceinline__ void attention_phase(const DecodeParams& D, const AttnParams& A, int n, unsigned char* smem_raw) {
    const int sub = threadIdx.x >> 7, tid = threadIdx.x & 127;
    if (sub >= 4) return;  // (THREADS is 512: never taken; keeps the mapping explicit)
    unsigned char* sm = smem_raw + (size_t)sub * D.att_item_bytes;
    const int ns = attn::attn_splits(A, n);
    const int n_items = D.n_kv * ns;
    for (int item = blockIdx.x * 4 + sub; item < n_items; item += gridDim.x * 4) {
        const int kvh = item / ns, split = item - kvh * ns;
        attn::attn_item<KV, MAXQ>(A, kvh, split, ns, n, tid, sm, 1 + sub);
        attn::att_sync(1 + sub);  // the item's shared memory is reused by the next one
    }
}

// The next layer's norm weights are read by every block of threads right after a barrier: pull them into L2
// while this layer runs (one 128-byte line per thread of one block of threads).
__device__ __forceinline__ void prefetch_norms(const DecodeParams& D, int l) {
    if (l >= D.n_layers || (int)blockIdx.x != l % (int)gridDim.x) return;
    const DecodeLayerPtrs& W = D.layer[l];
    const int lines = (D.dim * 4 + 127) >> 7;
    for (int i = threadIdx.x; i < 2 * lines; i += THREADS) {
        const char* p = reinterpret_cast<const char*>(i < lines ? W.attn_norm : W.ffn_norm) + (size_t)(i < lines ? i : i - lines) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
    }
}

template <class F, typename KV, int MAXQ>
__global__ void __launch_bounds__(THREADS, 1) decode_layers_kernel(const __grid_constant__ DecodeParams D) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Ring R;
    const LayerProg prog{D};
    ring_init(R, prog, D.dig_region, D.nstage, D.stage_stride, D.step_bytes, D.err_flag, D.wait_limit, smem_raw, threadIdx.x & 31, threadIdx.x >> 5);
    unsigned int epoch = 0;
    const int n_pos = __ldcg(D.d_pos) + 1;  // positions in the cache after this token (fixed for the launch)
    // One copy of the GEMV phase serves the four GEMVs of a layer (k = 0 QKV, 1 O, 2 gate/up, 3 down): the
    // code of a whole layer then fits the instruction cache and stays there from layer to layer.
    constexpr int PRO_MASK = (1 << PRO_NONE) | (1 << PRO_RMS);
    constexpr int EPI_MASK = (1 << EPI_QKV) | (1 << EPI_RESID) | (1 << EPI_SILU);
    for (int l = 0; l < D.n_layers; l++) {
        prefetch_norms(D, l + 1);
#pragma unroll 1
        for (int k = 0; k < 4; k++) {
            {
                GemvParams P = phase_params(D, l, k);
                P.pos1 = n_pos;
                const int nmat = k == 2 ? 2 : 1;
                const int pro = (k == 0 || k == 2) ? PRO_RMS : PRO_NONE;
                const int epi = k == 0 ? EPI_QKV : k == 2 ? EPI_SILU : EPI_RESID;
#ifndef SIZE_NO_GEMV
                gemv_phase<F, PRO_MASK, EPI_MASK>(P, R, prog, smem_raw, nmat, pro, epi);
#endif
            }
            if (k < 3 || l + 1 < D.n_layers) grid_sync(D, epoch);
            if (k == 0) {
                const AttnParams A = attn_params(D, l);
#ifndef SIZE_NO_ATTN
                attention_phase<KV, MAXQ>(D, A, n_pos, smem_raw);
#endif
                grid_sync(D, epoch);
            }
        }
    }
}

template <class F, typename KV, int MAXQ>
int launch_k(slai_ctx* ctx, const DecodeParams& D, size_t smem) {
    auto kern = decode_layers_kernel<F, KV, MAXQ>;
    static PerDeviceOnce attr;
    if (attr.need(ctx->device)) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
        attr.set(ctx->device);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx->sm_count);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;  // all blocks of threads resident together: the grid barrier needs it
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    SLAI_CHECK_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, D));
    return SLAI_OK;
}

template <class F>
int launch_f(slai_ctx* ctx, const DecodeParams& D, size_t smem) {
    const bool kv_f16 = D.kv_f16 != 0;
    if (D.kv_mul == 1) return kv_f16 ? launch_k<F, __half, 1>(ctx, D, smem) : launch_k<F, float, 1>(ctx, D, smem);
    return kv_f16 ? launch_k<F, __half, 8>(ctx, D, smem) : launch_k<F, float, 8>(ctx, D, smem);
}

}  // namespace

int decode_layers_prepare(slai_ctx* ctx, const DecodeLayersDesc& desc, DecodeLayersPlan* plan, DecodeParams* D) {
    // Common shared-memory geometry of all phases: the staging region must hold the widest activation vector
    // and four attention items; the ring depth follows from what is left.
    const int n_kv = desc.n_heads / desc.kv_mul;
    const int kv_dim = n_kv * desc.head_size;
    SLAI_REQUIRE(ctx, desc.dim % 16 == 0 && desc.hidden % 16 == 0 && kv_dim % 16 == 0, SLAI_ERR_SHAPE,
                 "decode: dimensions must be multiples of 16 for the fused path");
    const int esz = desc.kv_f16 ? 2 : 4;
    size_t dig = gemv_dig_region(desc.fmt, desc.dim);
    const size_t dig2 = gemv_dig_region(desc.fmt, desc.hidden);
    if (dig2 > dig) dig = dig2;
    // Attention runs four items per block of threads in the staging region plus the partial-sum buffer behind it
    // (both idle during that phase).  The tile shrinks until four items fit.
    int tile_pos = attn::attn_tile_pos(desc.head_size, esz);
    int n_splits = 0;
    size_t item_bytes = 0;
    for (;; tile_pos -= 8) {
        SLAI_REQUIRE(ctx, tile_pos >= 8, SLAI_ERR_SHAPE, "decode: attention items do not fit in shared memory");
        // one split per tile while they all run at once (four per block of threads); longer contexts walk several
        // tiles per split instead of queueing more splits
        n_splits = (desc.seq_len + tile_pos - 1) / tile_pos;
        const int at_once = (4 * ctx->sm_count) / n_kv;
        if (n_splits > at_once) n_splits = at_once < 1 ? 1 : at_once;
        if (n_splits > 64) n_splits = 64;
        item_bytes = attn::attn_item_bytes(desc.kv_mul, desc.head_size, esz, tile_pos, n_splits);
        if (4 * item_bytes <= dig + (size_t)RED_FLOATS * 4) break;
    }
    plan->dig_region = dig;
    plan->n_splits = n_splits;
    plan->part_o_bytes = (size_t)desc.n_heads * n_splits * desc.head_size * 4;
    plan->part_ml_bytes = (size_t)desc.n_heads * n_splits * 2 * 4;
    // ring depth: probe with the widest phase
    GemvLaunch L;
    L.fmt = desc.fmt;
    L.K = desc.hidden > desc.dim ? desc.hidden : desc.dim;
    L.nseg = 1;
    L.seg[0].rows = 16;
    L.seg[0].w = reinterpret_cast<const uint8_t*>(ctx->d_counters);  // only alignment is checked here
    L.v = reinterpret_cast<const float*>(ctx->d_counters);
    GemvParams P;
    size_t smem = 0;
    int rc = gemv_fill_params(ctx, L, dig, 0, P, &smem, nullptr);
    if (rc) return rc;
    plan->nstage = P.nstage;
    plan->smem = smem;
    D->fmt = desc.fmt; D->dim = desc.dim; D->hidden = desc.hidden; D->kv_dim = kv_dim; D->n_heads = desc.n_heads; D->n_kv = n_kv;
    D->kv_mul = desc.kv_mul; D->head_size = desc.head_size; D->seq_len = desc.seq_len;
    D->nsteps_dim = (int)layout::num_steps(desc.fmt, desc.dim);
    D->nsteps_hidden = (int)layout::num_steps(desc.fmt, desc.hidden);
    D->tile_bytes_dim = (long long)layout::tile_bytes(desc.fmt, desc.dim);
    D->tile_bytes_hidden = (long long)layout::tile_bytes(desc.fmt, desc.hidden);
    {
        const int G = ctx->sm_count;
        const int n_items[4] = {(desc.dim + 2 * kv_dim) / 16, desc.dim / 16, desc.hidden / 16, desc.dim / 16};
        for (int k = 0; k < 4; k++) {
            D->items_base[k] = n_items[k] / G;
            D->items_rem[k] = n_items[k] % G;
        }
    }
    D->nstage = P.nstage; D->step_bytes = P.step_bytes; D->stage_stride = P.stage_stride; D->dig_region = (int)dig;
    D->n_splits = n_splits; D->tile_pos = tile_pos; D->att_item_bytes = (int)item_bytes;
    D->bar = ctx->d_counters + CNT_GRID_BAR;
    D->err_flag = ctx->d_counters + CNT_ERR_FLAG;
    D->wait_limit = ctx->wait_limit;
    D->counters = ctx->d_counters;
    return SLAI_OK;
}

int decode_layers_launch(slai_ctx* ctx, const DecodeParams& D, const DecodeLayersPlan& plan) {
    SLAI_REQUIRE(ctx, D.n_layers >= 1 && D.n_layers <= DECODE_MAX_LAYERS, SLAI_ERR_SHAPE, "decode: %d layers (fused path holds up to %d)",
                 D.n_layers, DECODE_MAX_LAYERS);
    SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(D.bar, 0, sizeof(unsigned int), ctx->stream));
    switch (D.fmt) {
        case SLAI_FMT_Q4_K: return launch_f<Q4K>(ctx, D, plan.smem);
        case SLAI_FMT_Q5_K: return launch_f<Q5K>(ctx, D, plan.smem);
        case SLAI_FMT_Q6_K: return launch_f<Q6K>(ctx, D, plan.smem);
        case SLAI_FMT_Q8_0: return launch_f<Q80>(ctx, D, plan.smem);
    }
    return slai_set_error(ctx, SLAI_ERR_UNSUPPORTED_FORMAT, "decode: format %d has no fused kernel", D.fmt);
}

