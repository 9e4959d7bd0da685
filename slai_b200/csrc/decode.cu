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

struct DecodeParams {
    const GemvParams* prog;  // device array: 4 entries per layer (QKV, O, gate/up, down)
    const AttnParams* att;   // device array: one entry per layer
    int n_layers;
    int n_kv;                // KV heads
    int att_item_floats;     // shared-memory floats per attention item
    unsigned int* bar;       // grid barrier counter, zero at launch
    unsigned int* err_flag;
};

namespace {

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
            if (it > (1 << 22)) {
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
__device__ __forceinline__ void attention_phase(const DecodeParams& D, const AttnParams& A, unsigned char* smem_raw) {
    const int sub = threadIdx.x >> 7, tid = threadIdx.x & 127;
    if (sub >= 4) return;  // (THREADS is 512: never taken; keeps the mapping explicit)
    float* sm = reinterpret_cast<float*>(smem_raw) + (size_t)sub * D.att_item_floats;
    const int n_items = D.n_kv * A.n_splits;
    for (int item = blockIdx.x * 4 + sub; item < n_items; item += gridDim.x * 4) {
        const int kvh = item / A.n_splits, split = item - kvh * A.n_splits;
        attn::attn_item<KV, MAXQ>(A, kvh, split, tid, sm, 1 + sub);
        attn::att_sync(1 + sub);  // the item's shared memory is reused by the next one
    }
}

template <class F, typename KV, int MAXQ>
__global__ void __launch_bounds__(THREADS, 1) decode_layers_kernel(const __grid_constant__ DecodeParams D) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Ring R;
    ring_init(R, D.prog, 4 * D.n_layers, smem_raw, threadIdx.x & 31, threadIdx.x >> 5);
    unsigned int epoch = 0;
    for (int l = 0; l < D.n_layers; l++) {
        const GemvParams* pp = D.prog + 4 * l;
        gemv_phase<F, 1, PRO_RMS, EPI_QKV>(pp[0], R, smem_raw, l == 0);
        grid_sync(D, epoch);
        attention_phase<KV, MAXQ>(D, D.att[l], smem_raw);
        grid_sync(D, epoch);
        gemv_phase<F, 1, PRO_NONE, EPI_RESID>(pp[1], R, smem_raw, false);
        grid_sync(D, epoch);
        gemv_phase<F, 2, PRO_RMS, EPI_SILU>(pp[2], R, smem_raw, false);
        grid_sync(D, epoch);
        gemv_phase<F, 1, PRO_NONE, EPI_RESID>(pp[3], R, smem_raw, false);
        if (l + 1 < D.n_layers) grid_sync(D, epoch);
    }
}

template <class F, typename KV, int MAXQ>
int launch_k(slai_ctx* ctx, const DecodeParams& D, size_t smem) {
    auto kern = decode_layers_kernel<F, KV, MAXQ>;
    static bool attr_done = false;
    if (!attr_done) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
        attr_done = true;
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
int launch_f(slai_ctx* ctx, const DecodeParams& D, size_t smem, bool kv_f16, int kv_mul) {
    if (kv_mul == 1) return kv_f16 ? launch_k<F, __half, 1>(ctx, D, smem) : launch_k<F, float, 1>(ctx, D, smem);
    return kv_f16 ? launch_k<F, __half, 8>(ctx, D, smem) : launch_k<F, float, 8>(ctx, D, smem);
}

}  // namespace

int decode_layers_prepare(slai_ctx* ctx, const DecodeLayersDesc& desc, DecodeLayersPlan* plan) {
    // Common shared-memory geometry of all phases: the staging region must hold the widest activation vector
    // and four attention items; the ring depth follows from what is left.
    const int n_kv = desc.n_heads / desc.kv_mul;
    int n_splits = (4 * ctx->sm_count) / n_kv;
    if (n_splits > 64) n_splits = 64;
    if (n_splits > 2 * desc.head_size) n_splits = 2 * desc.head_size;
    if (n_splits < 1) n_splits = 1;
    while ((desc.seq_len + n_splits - 1) / n_splits > 1024) n_splits++;
    SLAI_REQUIRE(ctx, n_splits <= 2 * desc.head_size, SLAI_ERR_SHAPE, "decode: context too long for the fused path");
    const int chunk_max = (desc.seq_len + n_splits - 1) / n_splits;
    const size_t item_floats = (attn::attn_item_floats(desc.kv_mul, desc.head_size, chunk_max) + 3) & ~(size_t)3;
    size_t dig = gemv_dig_region(desc.fmt, desc.dim);
    const size_t dig2 = gemv_dig_region(desc.fmt, desc.hidden);
    if (dig2 > dig) dig = dig2;
    if (4 * item_floats * 4 > dig) dig = (4 * item_floats * 4 + 127) & ~(size_t)127;
    plan->dig_region = dig;
    plan->n_splits = n_splits;
    plan->chunk_max = chunk_max;
    plan->att_item_floats = (int)item_floats;
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
    return SLAI_OK;
}

int decode_layers_launch(slai_ctx* ctx, int fmt, const void* d_prog, const void* d_att, int n_layers, int n_kv, int kv_mul,
                         bool kv_f16, const DecodeLayersPlan& plan) {
    DecodeParams D;
    D.prog = reinterpret_cast<const GemvParams*>(d_prog);
    D.att = reinterpret_cast<const AttnParams*>(d_att);
    D.n_layers = n_layers;
    D.n_kv = n_kv;
    D.att_item_floats = plan.att_item_floats;
    D.bar = ctx->d_counters + 3100;
    D.err_flag = ctx->d_counters + 3000;
    SLAI_CHECK_CUDA(ctx, cudaMemsetAsync(D.bar, 0, sizeof(unsigned int), ctx->stream));
    switch (fmt) {
        case SLAI_FMT_Q4_K: return launch_f<Q4K>(ctx, D, plan.smem, kv_f16, kv_mul);
        case SLAI_FMT_Q5_K: return launch_f<Q5K>(ctx, D, plan.smem, kv_f16, kv_mul);
        case SLAI_FMT_Q6_K: return launch_f<Q6K>(ctx, D, plan.smem, kv_f16, kv_mul);
        case SLAI_FMT_Q8_0: return launch_f<Q80>(ctx, D, plan.smem, kv_f16, kv_mul);
    }
    return slai_set_error(ctx, SLAI_ERR_UNSUPPORTED_FORMAT, "decode: format %d has no fused kernel", fmt);
}

// Host-side builders used by model.cu (keep the parameter structs private to the CUDA files).
size_t decode_gemv_params_bytes() { return sizeof(GemvParams); }
size_t decode_attn_params_bytes() { return sizeof(AttnParams); }

int decode_fill_gemv(slai_ctx* ctx, const GemvLaunch& L, const DecodeLayersPlan& plan, void* h_out) {
    GemvParams P;
    int rc = gemv_fill_params(ctx, L, plan.dig_region, plan.nstage, P, nullptr, nullptr);
    if (rc) return rc;
    memcpy(h_out, &P, sizeof(P));
    return SLAI_OK;
}

void decode_fill_attn(slai_ctx* ctx, const DecodeLayersDesc& desc, const DecodeLayersPlan& plan, const float* q, const void* kc,
                      const void* vc, const int* d_pos, float* out, float* part_o, float* part_ml, void* h_out) {
    AttnParams A;
    A.q = q; A.kc = kc; A.vc = vc;
    A.pos_stride = desc.head_size; A.head_stride = (long long)desc.seq_len * desc.head_size;
    A.n_heads = desc.n_heads; A.kv_mul = desc.kv_mul; A.hs = desc.head_size;
    A.d_pos = d_pos; A.n_splits = plan.n_splits; A.chunk_max = plan.chunk_max;
    A.out = out; A.part_o = part_o; A.part_ml = part_ml;
    A.counters = ctx->d_counters;
    memcpy(h_out, &A, sizeof(A));
}
