// Fused dequant-GEMV for GGUF Q8_0 / Q4_K / Q5_K / Q6_K weights (GemvQuant::launch,
// crates/slai/src/ops/gemv_quant.rs:206-312) with the decode-path prologues and epilogues fused in:
//   prologue : none | RmsNorm (ops/rms_norm.rs:68-77) | LayerNorm+gamma/beta (ops/layernorm.rs:104-111)
//   epilogue : store | residual add | SiLU gate (ops/silu.rs:50-58) | GELU (ops/unary.rs:81-85) |
//              q/k/v split with RoPE (ops/rope.rs:88-125) and KV-cache append (transformer.rs:329-334)
//
// Kernel shape.  256 threads = 8 warps.  A work item is one 16-row tile; `KS` warps share an item and
// split its K range by steps, so a block works on 8/KS items at a time.  Every lane streams 16-byte
// chunks of packed quants straight from global memory (each row is read exactly once, 64 contiguous
// bytes per row per load instruction, two steps in flight per warp), expands them to exact f16 pairs
// and feeds mma.sync.m16n8k16 against the activation vector staged once per block in shared memory
// (see gemv_frag.cuh).  Scales are applied to the per-sub-block sums in f32; the lanes of a row are
// reduced by shuffles, the warps of an item through shared memory in a fixed order (deterministic).
//
// The first weight loads are issued before `griddepcontrol.wait`, so under programmatic dependent
// launch they overlap the tail of the kernel that produces the activation vector.
#include "common.cuh"
#include "gemv_frag.cuh"
#include "gemv_formats.cuh"

namespace {

using namespace frag;
using namespace gemvfmt;

constexpr int THREADS = 256;
constexpr int WARPS = 8;

struct GemvParams {
    GemvSeg seg[3];
    int nseg;
    int K;
    int n_items;     // 16-row tiles (NMAT==2: tiles of seg[0])
    int nsteps;      // K steps per row
    const float* v;
    float* out;
    const float* norm_w;
    const float* norm_b;
    float eps;
    const float* resid;
    int rope;
    const float* rope_theta;
    int head_size;
    const int* d_pos;
    void* kcache;
    void* vcache;
    int kv_f16;
    long long kv_pos_stride, kv_head_stride;
};

// ---------------------------------------------------------------------------------------------
// Block-wide reductions used by the staging pass.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
// returns (sum, max) over the block; `stat` is scratch of >= 2*WARPS floats
__device__ __forceinline__ void block_sum_max(float& s, float& m, float* stat) {
    s = warp_sum(s);
    m = warp_max(m);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) {
        stat[warp] = s;
        stat[WARPS + warp] = m;
    }
    __syncthreads();
    float ts = 0.f, tm = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; w++) {
        ts += stat[w];
        tm = fmaxf(tm, stat[WARPS + w]);
    }
    s = ts;
    m = tm;
}

// Stage the activation vector: optional normalisation, power-of-two scaling so that max|v| lands in
// [2^13, 2^14), split into f16 hi + lo in the [0,2,1,3] order, and per-32 sums of the scaled values
// (for the `- dmin*m * sum(v)` term of Q4_K / Q5_K).  Returns 1/scale.
template <int PRO, bool NEED_SV>
__device__ float stage_vector(const GemvParams& P, const Smem& S, int Kp) {
    const int K = P.K;
    const int tid = threadIdx.x;
    const float4* v4 = reinterpret_cast<const float4*>(P.v);
    const int n4 = K >> 2;  // K is a multiple of 32
    float mul = 1.f, sub = 0.f;
    float sum = 0.f, mx = 0.f;
    if (PRO == PRO_LN) {
        for (int i = tid; i < n4; i += THREADS) {
            const float4 x = __ldg(v4 + i);
            sum += (x.x + x.y) + (x.z + x.w);
        }
        block_sum_max(sum, mx, S.stat);
        sub = sum / (float)K;
        sum = 0.f;
    }
    const float4* w4p = reinterpret_cast<const float4*>(P.norm_w);
    const float4* b4p = reinterpret_cast<const float4*>(P.norm_b);
    for (int i = tid; i < n4; i += THREADS) {
        float4 x = __ldg(v4 + i);
        if (PRO == PRO_NONE) {
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
        } else if (PRO == PRO_RMS) {
            const float4 w = __ldg(w4p + i);
            sum += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(x.x * w.x), fabsf(x.y * w.y)), fmaxf(fabsf(x.z * w.z), fabsf(x.w * w.w))));
        } else {
            const float4 w = __ldg(w4p + i);
            x.x -= sub; x.y -= sub; x.z -= sub; x.w -= sub;
            sum += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(x.x * w.x), fabsf(x.y * w.y)), fmaxf(fabsf(x.z * w.z), fabsf(x.w * w.w))));
        }
    }
    block_sum_max(sum, mx, S.stat);
    if (PRO == PRO_RMS) {
        mul = 1.0f / sqrtf(sum / (float)K + P.eps);
        mx *= mul;
    } else if (PRO == PRO_LN) {
        mul = 1.0f / sqrtf(sum / (float)K + P.eps);
        mx *= mul;
        if (P.norm_b) {
            float mb = 0.f, dummy = 0.f;
            for (int i = tid; i < n4; i += THREADS) {
                const float4 b = __ldg(b4p + i);
                mb = fmaxf(mb, fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
            }
            block_sum_max(dummy, mb, S.stat);
            mx += mb;
        }
    }
    // power-of-two scale: max|v| * scale in [2^13, 2^14)
    float scale = 1.f;
    if (mx > 0.f && mx < 3.0e38f) {
        int e;
        frexpf(mx, &e);  // mx = f * 2^e, f in [0.5, 1)
        e = e < -100 ? -100 : e;
        scale = ldexpf(1.0f, 14 - e);
    }
    __half* hi = reinterpret_cast<__half*>(__cvta_shared_to_generic(S.hi));
    __half* lo = reinterpret_cast<__half*>(__cvta_shared_to_generic(S.lo));
    const int np4 = Kp >> 2;
    for (int i = tid; i < np4; i += THREADS) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            x = __ldg(v4 + i);
            if (PRO == PRO_RMS) {
                const float4 w = __ldg(w4p + i);
                x.x = (x.x * mul) * w.x; x.y = (x.y * mul) * w.y; x.z = (x.z * mul) * w.z; x.w = (x.w * mul) * w.w;
            } else if (PRO == PRO_LN) {
                const float4 w = __ldg(w4p + i);
                x.x = ((x.x - sub) * mul) * w.x; x.y = ((x.y - sub) * mul) * w.y;
                x.z = ((x.z - sub) * mul) * w.z; x.w = ((x.w - sub) * mul) * w.w;
                if (P.norm_b) {
                    const float4 b = __ldg(b4p + i);
                    x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
                }
            }
            x.x *= scale; x.y *= scale; x.z *= scale; x.w *= scale;
        }
        const __half h0 = __float2half_rn(x.x), h1 = __float2half_rn(x.y), h2 = __float2half_rn(x.z), h3 = __float2half_rn(x.w);
        const __half l0 = __float2half_rn(x.x - __half2float(h0)), l1 = __float2half_rn(x.y - __half2float(h1));
        const __half l2 = __float2half_rn(x.z - __half2float(h2)), l3 = __float2half_rn(x.w - __half2float(h3));
        // order [0,2,1,3]
        __half2* hp = reinterpret_cast<__half2*>(hi + 4 * i);
        __half2* lp = reinterpret_cast<__half2*>(lo + 4 * i);
        hp[0] = __halves2half2(h0, h2);
        hp[1] = __halves2half2(h1, h3);
        lp[0] = __halves2half2(l0, l2);
        lp[1] = __halves2half2(l1, l3);
        if (NEED_SV) {
            float s4 = (x.x + x.y) + (x.z + x.w);
            s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
            s4 += __shfl_xor_sync(0xffffffffu, s4, 2);
            s4 += __shfl_xor_sync(0xffffffffu, s4, 4);
            if ((tid & 7) == 0) reinterpret_cast<float*>(__cvta_shared_to_generic(S.sv))[i >> 3] = s4;
        }
    }
    if (tid < 8) reinterpret_cast<uint32_t*>(__cvta_shared_to_generic(S.zero))[tid] = 0u;
    __syncthreads();
    return 1.0f / scale;
}

__device__ __forceinline__ float gelu_ref(float x) {
    const float A = 0.044715f, Sq = 0.7978846f;
    return 0.5f * x * (1.0f + tanhf(Sq * x * (1.0f + A * x * x)));
}

__device__ __forceinline__ int seg_of_tile(const GemvParams& P, int tile) {
    int s = 0;
    if (P.nseg > 1 && tile >= P.seg[1].tile0) s = 1;
    if (P.nseg > 2 && tile >= P.seg[2].tile0) s = 2;
    return s;
}

// ---------------------------------------------------------------------------------------------
// The kernel.
// ---------------------------------------------------------------------------------------------
template <class F, int KS, int NMAT, int PRO, int EPI>
__global__ void __launch_bounds__(THREADS, 2) gemv_kernel(const GemvParams P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = P.K;
    const int Kp = (K + 255) & ~255;
    Smem S;
    S.hi = (uint32_t)__cvta_generic_to_shared(smem_raw);
    S.lo = S.hi + 2 * Kp;
    S.zero = S.lo + 2 * Kp;
    S.sv = S.zero + 32;
    S.red = reinterpret_cast<float*>(smem_raw + 4 * Kp + 32) + (Kp >> 5);
    S.stat = S.red + WARPS * 32;

    LaneCtx L;
    L.lane = threadIdx.x & 31;
    L.g = L.lane >> 2;
    L.t = L.lane & 3;
    for (int i = 0; i < 8; i++) { L.bp[i] = 0; L.bs[i] = 0; }
    F::init(L, S);
    L.bs[7] = F::aux(K);

    constexpr int GROUPS = WARPS / KS;
    const int warp = threadIdx.x >> 5;
    const int grp = warp / KS, wi = warp % KS;
    const int item_stride = gridDim.x * GROUPS;
    int item = blockIdx.x * GROUPS + grp;
    const int nsteps = P.nsteps;

    typename F::Regs R0, R1;
    const uint8_t *rowA = nullptr, *rowB = nullptr;
    auto rows_of = [&](int it, int mat) {
        int s = NMAT == 2 ? mat : seg_of_tile(P, it);
        const int tile_in_seg = NMAT == 2 ? it : it - P.seg[s].tile0;
        const uint8_t* base = P.seg[s].w + (size_t)(tile_in_seg * 16 + L.g) * P.seg[s].row_stride;
        rowA = base;
        rowB = base + 8 * P.seg[s].row_stride;
    };
    // First loads before waiting for the producer of `v`.
    bool preloaded = false;
    if (item < P.n_items && wi < nsteps) {
        rows_of(item, 0);
        F::load(R0, rowA, rowB, wi, L);
        preloaded = true;
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float inv_scale = stage_vector<PRO, F::NEED_SV>(P, S, Kp);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    for (; item < P.n_items; item += item_stride) {
        float acc[NMAT][2];
#pragma unroll
        for (int mat = 0; mat < NMAT; mat++) {
            acc[mat][0] = 0.f;
            acc[mat][1] = 0.f;
            rows_of(item, mat);
            int s = wi;
            if (s < nsteps) {
                if (!preloaded) F::load(R0, rowA, rowB, s, L);
                preloaded = false;
                while (true) {
                    if (s + KS < nsteps) F::load(R1, rowA, rowB, s + KS, L);
                    F::compute(R0, s, L, S, acc[mat][0], acc[mat][1]);
                    s += KS;
                    if (s >= nsteps) break;
                    if (s + KS < nsteps) F::load(R0, rowA, rowB, s + KS, L);
                    F::compute(R1, s, L, S, acc[mat][0], acc[mat][1]);
                    s += KS;
                    if (s >= nsteps) break;
                }
            }
            // reduce the four lanes that share a row
            acc[mat][0] += __shfl_xor_sync(0xffffffffu, acc[mat][0], 1);
            acc[mat][0] += __shfl_xor_sync(0xffffffffu, acc[mat][0], 2);
            acc[mat][1] += __shfl_xor_sync(0xffffffffu, acc[mat][1], 1);
            acc[mat][1] += __shfl_xor_sync(0xffffffffu, acc[mat][1], 2);
        }
        // partials of this warp: red[warp][mat*16 + row]
        float* my = S.red + warp * 32;
        if (L.t == 0) {
#pragma unroll
            for (int mat = 0; mat < NMAT; mat++) {
                my[mat * 16 + L.g] = acc[mat][0];
                my[mat * 16 + L.g + 8] = acc[mat][1];
            }
        }
        if (KS == 1) {
            __syncwarp();
        } else if (KS == WARPS) {
            __syncthreads();
        } else {
            asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(KS * 32) : "memory");
        }
        if (wi == 0 && L.lane < 16) {
            const int r = L.lane;
            float val[NMAT];
#pragma unroll
            for (int mat = 0; mat < NMAT; mat++) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < KS; w++) s += S.red[(grp * KS + w) * 32 + mat * 16 + r];
                val[mat] = s * inv_scale;
            }
            const int sidx = NMAT == 2 ? 0 : seg_of_tile(P, item);
            const GemvSeg& sg = P.seg[sidx];
            const int row_in_seg = (NMAT == 2 ? item : item - sg.tile0) * 16 + r;
            const bool valid = row_in_seg < sg.rows;
            const int orow = sg.out_off + row_in_seg;
            const float bias = (sg.bias && valid) ? sg.bias[row_in_seg] : 0.f;
            if (EPI == EPI_STORE) {
                if (valid) P.out[orow] = val[0] + bias;
            } else if (EPI == EPI_RESID) {
                if (valid) P.out[orow] = P.resid[orow] + (val[0] + bias);
            } else if (EPI == EPI_SILU) {
                if (valid) {
                    const float gt = val[0], up = val[NMAT - 1];
                    P.out[orow] = up * (gt / (1.0f + expf(-gt)));
                }
            } else if (EPI == EPI_GELU) {
                if (valid) P.out[orow] = gelu_ref(val[0] + bias);
            } else if (EPI == EPI_QKV) {
                float y = val[0] + bias;
                const int pos = *P.d_pos;
                if (P.rope && sg.role < 2) {
                    const float other = __shfl_xor_sync(0x0000ffffu, y, 1);
                    const int hd = (row_in_seg & ~1) % P.head_size;
                    const float ang = (float)pos * P.rope_theta[hd >> 1];
                    float sn, cs;
                    sincosf(ang, &sn, &cs);
                    y = (r & 1) ? (sn * other + cs * y) : (cs * y - sn * other);
                }
                if (valid) {
                    if (sg.role == 0) {
                        P.out[orow] = y;
                    } else {
                        void* cache = sg.role == 1 ? P.kcache : P.vcache;
                        const int head = row_in_seg / P.head_size, d = row_in_seg % P.head_size;
                        const long long off = (long long)pos * P.kv_pos_stride + (long long)head * P.kv_head_stride + d;
                        if (P.kv_f16) reinterpret_cast<__half*>(cache)[off] = __float2half_rn(y);
                        else reinterpret_cast<float*>(cache)[off] = y;
                    }
                }
            }
        }
        // the partial buffer is reused by the next item of this group
        if (KS == 1) {
            __syncwarp();
        } else if (KS == WARPS) {
            __syncthreads();
        } else {
            asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(KS * 32) : "memory");
        }
    }
}

// Dense f32 matrix (GpuQuantMatrix::F32): one warp per row.
__global__ void gemv_f32_kernel(float* out, const float* w, const float* v, int M, int K, long long row_stride_f) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= M) return;
    const float* wr = w + (size_t)row * row_stride_f;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(wr[k], v[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) out[row] = acc;
}

template <class F, int KS, int NMAT, int PRO, int EPI>
int launch_inst(slai_ctx* ctx, const GemvParams& P, int grid, size_t smem, bool pdl) {
    auto kern = gemv_kernel<F, KS, NMAT, PRO, EPI>;
    static bool attr_done = false;  // per instantiation
    if (!attr_done) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_done = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
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

template <class F, int NMAT, int PRO, int EPI>
int launch_ks(slai_ctx* ctx, const GemvParams& P, int ks, int grid_cap, size_t smem, bool pdl) {
    auto grid_for = [&](int k) {
        const int groups = WARPS / k;
        int g = (P.n_items + groups - 1) / groups;
        return g < grid_cap ? g : grid_cap;
    };
    switch (ks) {
        case 1: return launch_inst<F, 1, NMAT, PRO, EPI>(ctx, P, grid_for(1), smem, pdl);
        case 2: return launch_inst<F, 2, NMAT, PRO, EPI>(ctx, P, grid_for(2), smem, pdl);
        case 4: return launch_inst<F, 4, NMAT, PRO, EPI>(ctx, P, grid_for(4), smem, pdl);
        default: return launch_inst<F, 8, NMAT, PRO, EPI>(ctx, P, grid_for(8), smem, pdl);
    }
}

template <class F>
int launch_fmt(slai_ctx* ctx, const GemvParams& P, const GemvLaunch& L, int ks, int grid_cap, size_t smem) {
    const bool pdl = L.pdl;
#define GO(NMAT, PRO, EPI) return launch_ks<F, NMAT, PRO, EPI>(ctx, P, ks, grid_cap, smem, pdl)
    switch (L.epi) {
        case EPI_STORE:
            if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_STORE);
            if (L.pro == PRO_RMS) GO(1, PRO_RMS, EPI_STORE);
            GO(1, PRO_LN, EPI_STORE);
        case EPI_RESID:
            if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_RESID);
            break;
        case EPI_SILU:
            if (L.pro == PRO_RMS) GO(2, PRO_RMS, EPI_SILU);
            if (L.pro == PRO_NONE) GO(2, PRO_NONE, EPI_SILU);
            break;
        case EPI_GELU:
            if (L.pro == PRO_LN) GO(1, PRO_LN, EPI_GELU);
            if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_GELU);
            break;
        case EPI_QKV:
            if (L.pro == PRO_RMS) GO(1, PRO_RMS, EPI_QKV);
            if (L.pro == PRO_LN) GO(1, PRO_LN, EPI_QKV);
            if (L.pro == PRO_NONE) GO(1, PRO_NONE, EPI_QKV);
            break;
    }
#undef GO
    return slai_set_error(ctx, SLAI_ERR_INVALID_ARG, "gemv: unsupported prologue/epilogue combination %d/%d", L.pro, L.epi);
}

}  // namespace

int gemv_launch(slai_ctx* ctx, const GemvLaunch& L) {
    const int K = L.K;
    if (L.fmt == SLAI_FMT_F32) {
        SLAI_REQUIRE(ctx, L.nseg == 1 && L.pro == PRO_NONE && L.epi == EPI_STORE && !L.seg[0].bias, SLAI_ERR_INVALID_ARG,
                     "gemv: dense f32 matrices support only the plain product");
        const int M = L.seg[0].rows;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((M + 7) / 8);
        cfg.blockDim = dim3(256);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = L.pdl ? 1 : 0;
        SLAI_CHECK_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_f32_kernel, L.out, (const float*)L.seg[0].w, L.v, M, K,
                                                (long long)(L.seg[0].row_stride / 4)));
        return SLAI_OK;
    }
    const int be = fmt_block_elems(L.fmt);
    SLAI_REQUIRE(ctx, be > 0 && L.fmt != SLAI_FMT_F32, SLAI_ERR_UNSUPPORTED_FORMAT, "gemv: format %d has no kernel", L.fmt);
    SLAI_REQUIRE(ctx, K > 0 && K % be == 0, SLAI_ERR_SHAPE, "gemv: K=%d is not a multiple of the block size %d", K, be);
    SLAI_REQUIRE(ctx, ((uintptr_t)L.v & 15) == 0, SLAI_ERR_INVALID_ARG, "gemv: input vector must be 16-byte aligned");

    GemvParams P = {};
    P.nseg = L.nseg;
    int tiles = 0;
    for (int s = 0; s < L.nseg; s++) {
        P.seg[s] = L.seg[s];
        P.seg[s].tile0 = tiles;
        tiles += (L.seg[s].rows + 15) / 16;
    }
    const bool dual = (L.epi == EPI_SILU);
    if (dual) {
        SLAI_REQUIRE(ctx, L.nseg == 2 && L.seg[0].rows == L.seg[1].rows, SLAI_ERR_SHAPE, "gemv: gate/up shapes differ");
        P.n_items = (L.seg[0].rows + 15) / 16;
    } else {
        P.n_items = tiles;
    }
    if (L.epi == EPI_QKV) {
        SLAI_REQUIRE(ctx, L.head_size > 0 && L.head_size % 2 == 0 && L.d_pos, SLAI_ERR_INVALID_ARG, "gemv: bad q/k/v arguments");
        SLAI_REQUIRE(ctx, !L.rope || L.rope_theta, SLAI_ERR_INVALID_ARG, "gemv: RoPE table missing");
    }
    P.K = K;
    const int step = (L.fmt == SLAI_FMT_Q4_K || L.fmt == SLAI_FMT_Q5_K) ? 256 : 128;
    P.nsteps = (K + step - 1) / step;
    P.v = L.v; P.out = L.out; P.norm_w = L.norm_w; P.norm_b = L.norm_b; P.eps = L.eps;
    P.resid = L.resid; P.rope = L.rope; P.rope_theta = L.rope_theta; P.head_size = L.head_size;
    P.d_pos = L.d_pos; P.kcache = L.kcache; P.vcache = L.vcache; P.kv_f16 = (L.kv_dtype == SLAI_KV_F16);
    P.kv_pos_stride = L.kv_pos_stride; P.kv_head_stride = L.kv_head_stride;

    const int Kp = (K + 255) & ~255;
    const size_t smem = (size_t)4 * Kp + 32 + (size_t)(Kp / 32) * 4 + WARPS * 32 * 4 + 64 * 4;
    SLAI_REQUIRE(ctx, smem <= 200 * 1024, SLAI_ERR_SHAPE, "gemv: K=%d needs %zu bytes of shared memory (max 204800)", K, smem);

    // K split: enough warp-items to fill the machine, at least two steps per warp where possible.
    static int ks_env = -1;
    if (ks_env < 0) {
        const char* e = getenv("SLAI_GEMV_KS");
        ks_env = e ? atoi(e) : 0;
    }
    int ks = 8;
    const double want = 1.5 * ctx->sm_count * 16.0 / (double)(P.n_items * (dual ? 2 : 1));
    while (ks > 1 && ks > want) ks >>= 1;
    while (ks > 1 && P.nsteps < ks) ks >>= 1;
    if (ks_env == 1 || ks_env == 2 || ks_env == 4 || ks_env == 8) ks = ks_env;
    const int ctas_per_sm = smem > 100 * 1024 ? 1 : 2;
    const int grid_cap = ctx->sm_count * ctas_per_sm;

    switch (L.fmt) {
        case SLAI_FMT_Q4_K: return launch_fmt<Q4K>(ctx, P, L, ks, grid_cap, smem);
        case SLAI_FMT_Q5_K: return launch_fmt<Q5K>(ctx, P, L, ks, grid_cap, smem);
        case SLAI_FMT_Q6_K: return launch_fmt<Q6K>(ctx, P, L, ks, grid_cap, smem);
        case SLAI_FMT_Q8_0: return launch_fmt<Q80>(ctx, P, L, ks, grid_cap, smem);
    }
    return slai_set_error(ctx, SLAI_ERR_UNSUPPORTED_FORMAT, "gemv: format %d has no kernel", L.fmt);
}
