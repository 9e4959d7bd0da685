// Fused dequant-GEMV for GGUF Q8_0 / Q4_K / Q5_K / Q6_K weights (GemvQuant::launch,
// crates/slai/src/ops/gemv_quant.rs:206-312) with the decode-path prologues and epilogues fused in:
//   prologue : none | RmsNorm (ops/rms_norm.rs:68-77) | LayerNorm+gamma/beta (ops/layernorm.rs:104-111)
//   epilogue : store | residual add | SiLU gate (ops/silu.rs:50-58) | GELU (ops/unary.rs:81-85) |
//              q/k/v split with RoPE (ops/rope.rs:88-125) and KV-cache append (transformer.rs:329-334)
//
// Kernel shape.  One persistent block of 16 warps per SM.  The weights are stored tile-major (layout.cuh):
// the packed data of 16 rows x one K step is one contiguous block.  Work is divided in two levels so that
// every SM and every warp gets the same amount (+-1 block) whatever the matrix shape: the 16-row tiles are
// dealt out in contiguous, equal runs to the thread blocks; inside a block of threads the run's sequence of
// (tile, matrix, K-step) units is cut into 16 equal contiguous pieces, one per warp.  A warp's piece may
// cover the end of one tile and the start of the next; its partial row sums go to shared memory, and after
// a barrier the 16 partials of every row are added in warp order (deterministic) and the epilogue runs.
//
// Data movement: every warp owns a private ring of shared-memory stages; one lane issues a bulk asynchronous
// copy (cp.async.bulk, completion counted on an mbarrier) per block, always NSTAGE blocks ahead of the block
// being consumed, so the bytes in flight per SM are set by the ring size (100-180 KB), not by registers or
// occupancy.  Arithmetic: packed quants, four per register, go to the integer tensor-core MMA
// (mma.sync.m16n8k32 s8) against base-128 digit planes of the activation vector, staged once per block of
// threads in shared memory (gemv_frag.cuh); block scales are applied to the per-sub-block integer sums.
//
// Every mbarrier wait is bounded; on expiry the warp raises the context's error flag and stops waiting.
#include "common.cuh"
#include "gemv_frag.cuh"
#include "gemv_formats.cuh"
#include "layout.cuh"

namespace {

using namespace frag;
using namespace gemvfmt;

#ifndef SLAI_GEMV_WARPS
#define SLAI_GEMV_WARPS 16
#endif
constexpr int WARPS = SLAI_GEMV_WARPS;
constexpr int THREADS = 32 * WARPS;
constexpr int MAX_STAGES = 8;
constexpr int WAVE = 8;  // tiles whose partial sums are held in shared memory at a time
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int STAGE_REGS = 6;  // float4 per thread kept in registers between the staging passes (K <= 12288)

struct GemvParams {
    GemvSeg seg[3];
    int nseg;
    int K;
    int n_items;     // 16-row tiles (dual launch: tiles of seg[0])
    int nsteps;      // tile-step blocks per tile
    int nstage;      // ring depth per warp
    int step_bytes;  // bytes of a tile-step block
    int stage_stride;
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
    unsigned int* err_flag;
#ifdef SLAI_TRACE
    unsigned long long* trace;  // debug build only: per block of threads 8 x (globaltimer, clock64)
#endif
};

#ifdef SLAI_TRACE
#define SLAI_TRACE_POINT(k)                                                                     \
    if (threadIdx.x == 0 && P.trace) {                                                           \
        unsigned long long gt;                                                                   \
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));                                    \
        P.trace[(blockIdx.x * 8 + (k)) * 2] = gt;                                                \
        P.trace[(blockIdx.x * 8 + (k)) * 2 + 1] = (unsigned long long)clock64();                 \
    }
#else
#define SLAI_TRACE_POINT(k)
#endif

// ---- mbarrier / bulk copy -------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t a, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and raises the error flag) if the phase does not complete.
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity, unsigned int* err_flag) {
    for (int i = 0; i < (1 << 20); i++) {
        if (mbar_try_wait(a, parity)) return true;
        if (i > 1024) __nanosleep(64);
    }
    atomicExch(err_flag, 1u);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(mbar)
                 : "memory");
}

// ---- block-wide reductions used by the staging pass -----------------------------------------
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

__device__ __forceinline__ float max4(const float4& x) { return fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))); }

// Stage the activation vector: optional normalisation, power-of-two scaling so that max|v| lands in
// [2^25, 2^26), rounding to integers, split into four base-128 digit planes (gemv_frag.cuh), and per-sub-block
// digit sums (for the `- dmin*m * sum(v)` term of Q4_K / Q5_K and the -32 offset of Q6_K).  Returns 1/scale.
// The vector is read from global memory once and kept in registers between the passes when K <= 12288.
template <int PRO, int SV_GRAN, bool CACHED, class Hook>
__device__ float stage_impl(const GemvParams& P, const Smem& S, float* stat, int Kp, Hook after_loads) {
    const int K = P.K;
    const int tid = threadIdx.x;
    const float4* v4 = reinterpret_cast<const float4*>(P.v);
    const float4* w4p = reinterpret_cast<const float4*>(P.norm_w);
    const float4* b4p = reinterpret_cast<const float4*>(P.norm_b);
    const int n4 = K >> 2, np4 = Kp >> 2;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 xr[CACHED ? STAGE_REGS : 1];
    if (CACHED) {
#pragma unroll
        for (int r = 0; r < STAGE_REGS; r++) {
            const int i = tid + r * THREADS;
            xr[r] = i < n4 ? __ldg(v4 + i) : zero4;
        }
    }
    after_loads();  // the vector's loads are in flight ahead of whatever this issues
    // element group of register slot r (CACHED) or of loop round r (not CACHED)
#define SLAI_STAGE_LOOP(...)                                                            \
    if (CACHED) {                                                                       \
        _Pragma("unroll") for (int r = 0; r < STAGE_REGS; r++) {                        \
            const int i = tid + r * THREADS;                                            \
            float4 x = xr[r];                                                           \
            __VA_ARGS__                                                                    \
        }                                                                               \
    } else {                                                                            \
        for (int i = tid; i < np4; i += THREADS) {                                      \
            float4 x = i < n4 ? __ldg(v4 + i) : zero4;                                  \
            __VA_ARGS__                                                                    \
        }                                                                               \
    }
    float mul = 1.f, sub = 0.f;
    float sum = 0.f, mx = 0.f;
    if (PRO == PRO_LN) {
        SLAI_STAGE_LOOP({ sum += (x.x + x.y) + (x.z + x.w); })
        block_sum_max(sum, mx, stat);
        sub = sum / (float)K;
        sum = 0.f;
    }
    SLAI_STAGE_LOOP({
        if (i < n4) {
            if (PRO == PRO_NONE) {
                mx = fmaxf(mx, max4(x));
            } else {
                const float4 w = __ldg(w4p + i);
                if (PRO == PRO_LN) { x.x -= sub; x.y -= sub; x.z -= sub; x.w -= sub; }
                sum += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
                mx = fmaxf(mx, max4(make_float4(x.x * w.x, x.y * w.y, x.z * w.z, x.w * w.w)));
            }
        }
    })
    block_sum_max(sum, mx, stat);
    if (PRO != PRO_NONE) {
        mul = 1.0f / sqrtf(sum / (float)K + P.eps);
        mx *= mul;
        if (PRO == PRO_LN && P.norm_b) {
            float mb = 0.f, dummy = 0.f;
            for (int i = tid; i < n4; i += THREADS) mb = fmaxf(mb, max4(__ldg(b4p + i)));
            block_sum_max(dummy, mb, stat);
            mx += mb;
        }
    }
    float scale = 1.f;
    if (mx > 0.f && mx < 3.0e38f) {
        int e;
        frexpf(mx, &e);  // mx = f * 2^e, f in [0.5, 1)
        e = e < -90 ? -90 : e;
        scale = ldexpf(1.0f, 26 - e);
    }
    unsigned char* dig = reinterpret_cast<unsigned char*>(__cvta_shared_to_generic(S.dig));
    int4* sv = reinterpret_cast<int4*>(__cvta_shared_to_generic(S.sv));
    SLAI_STAGE_LOOP({
        if (i < np4) {  // np4 is a multiple of 64: whole warps take the branch together
            if (i < n4) {
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
            }
            int d0[4], d1[4], d2[4], d3[4];
            split_digits(__float2int_rn(x.x * scale), d0);
            split_digits(__float2int_rn(x.y * scale), d1);
            split_digits(__float2int_rn(x.z * scale), d2);
            split_digits(__float2int_rn(x.w * scale), d3);
            int s[4];
            _Pragma("unroll") for (int p = 0; p < 4; p++) {
                const uint32_t word = (uint32_t)(d0[p] & 0xFF) | ((uint32_t)(d1[p] & 0xFF) << 8) | ((uint32_t)(d2[p] & 0xFF) << 16) |
                                      ((uint32_t)(d3[p] & 0xFF) << 24);
                *reinterpret_cast<uint32_t*>(dig + (size_t)p * S.plane + 4 * i) = word;
                s[p] = (d0[p] + d1[p]) + (d2[p] + d3[p]);
            }
            if (SV_GRAN > 0) {
                _Pragma("unroll") for (int p = 0; p < 4; p++) {
                    s[p] += __shfl_xor_sync(0xffffffffu, s[p], 1);
                    s[p] += __shfl_xor_sync(0xffffffffu, s[p], 2);
                    if (SV_GRAN == 32) s[p] += __shfl_xor_sync(0xffffffffu, s[p], 4);
                }
                constexpr int LANES = SV_GRAN > 0 ? SV_GRAN / 4 : 1;  // float4 groups per sub-block
                if ((tid & (LANES - 1)) == 0) sv[i / LANES] = make_int4(s[0], s[1], s[2], s[3]);
            }
        }
    })
#undef SLAI_STAGE_LOOP
    __syncthreads();
    return 1.0f / scale;
}

template <int PRO, int SV_GRAN, class Hook>
__device__ float stage_vector(const GemvParams& P, const Smem& S, float* stat, int Kp, Hook after_loads) {
    if ((Kp >> 2) <= STAGE_REGS * THREADS) return stage_impl<PRO, SV_GRAN, true>(P, S, stat, Kp, after_loads);
    return stage_impl<PRO, SV_GRAN, false>(P, S, stat, Kp, after_loads);
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
template <class F, int NMAT, int PRO, int EPI>
__global__ void __launch_bounds__(THREADS, 1) gemv_kernel(const GemvParams P) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int K = P.K;
    const int Kp = (K + 255) & ~255;
    // [digit planes 4*(Kp+32) s8][sv: Kp/SV_GRAN x 4 s32][red WAVE*WARPS*NMAT*16 f32][stat 64 f32]
    // [mbar WARPS*MAX_STAGES u64][ring]
    constexpr int SV_BYTES_PER_256 = F::SV_GRAN > 0 ? 256 / F::SV_GRAN * 16 : 0;
    constexpr int RED_FLOATS = WAVE * WARPS * NMAT * 16;
    const uint32_t sv_bytes = (uint32_t)(Kp >> 8) * SV_BYTES_PER_256;
    Smem S;
    S.dig = (uint32_t)__cvta_generic_to_shared(smem_raw);
    S.plane = Kp + 32;  // planes 32 bytes apart modulo 128: the four digit columns of a sub-block hit different banks
    S.sv = S.dig + 4 * S.plane;
    float* red = reinterpret_cast<float*>(smem_raw + 4 * S.plane + sv_bytes);
    float* stat = red + RED_FLOATS;
    const uint32_t fixed = (uint32_t)(4 * S.plane) + sv_bytes + RED_FLOATS * 4 + 64 * 4;
    const uint32_t mbar_base = S.dig + fixed;
    const uint32_t ring_base = (mbar_base + WARPS * MAX_STAGES * 8 + 127u) & ~127u;

    const int tid = threadIdx.x, warp = tid >> 5;
    SLAI_TRACE_POINT(0)
    LaneCtx L;
    lane_init(L, tid & 31, S);

    // Work of this block of threads: tiles [i0, i1); in waves of WAVE tiles the units (tile, matrix, step) are cut
    // into WARPS contiguous pieces.
    const int nstage = P.nstage, nsteps = P.nsteps;
    const int upi = nsteps * NMAT;  // units per tile
    const int i0 = (int)(((long long)P.n_items * blockIdx.x) / gridDim.x);
    const int i1 = (int)(((long long)P.n_items * (blockIdx.x + 1)) / gridDim.x);
    const int n_local = i1 - i0;
    const int n_waves = (n_local + WAVE - 1) / WAVE;
    auto wave_range = [&](int wv, int& u0, int& u1) {  // this warp's unit range inside wave wv
        const int items = min(WAVE, n_local - wv * WAVE);
        const int U = items * upi;
        u0 = (U * warp) / WARPS;
        u1 = (U * (warp + 1)) / WARPS;
    };
    const uint32_t my_mbar = mbar_base + warp * MAX_STAGES * 8;
    const uint32_t my_ring = ring_base + warp * nstage * P.stage_stride;

    if (L.lane == 0) {
        for (int s = 0; s < nstage; s++) mbar_init(my_mbar + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // Producer cursor: (wave, unit) in the same order the consumer walks; the source pointer is advanced
    // incrementally (divisions only when a wave starts).
    int p_wave = 0, p_u = 0, p_u1 = 0, p_stage = 0, p_li = 0, p_mat = 0, p_step = 0;
    const uint8_t* p_ptr = nullptr;
    auto p_base = [&](int li, int mat) -> const uint8_t* {
        const int item = i0 + p_wave * WAVE + li;
        const int sidx = NMAT == 2 ? mat : seg_of_tile(P, item);
        const GemvSeg& sg = P.seg[sidx];
        const int tile = NMAT == 2 ? item : item - sg.tile0;
        return sg.w + (size_t)tile * sg.tile_bytes;
    };
    auto p_seek = [&]() {
        if (p_u < p_u1) {
            p_li = p_u / upi;
            const int rem = p_u - p_li * upi;
            p_mat = NMAT == 2 ? rem / nsteps : 0;
            p_step = rem - p_mat * nsteps;
            p_ptr = p_base(p_li, p_mat) + (size_t)p_step * P.step_bytes;
        }
    };
    if (n_waves > 0) {
        wave_range(0, p_u, p_u1);
        p_seek();
    }
    auto issue = [&]() {
        while (p_wave < n_waves && p_u >= p_u1) {  // skip empty ranges, move to the next wave
            if (++p_wave < n_waves) {
                wave_range(p_wave, p_u, p_u1);
                p_seek();
            }
        }
        if (p_wave < n_waves) {
            if (L.lane == 0) {
                const uint32_t mb = my_mbar + 8 * p_stage;
                mbar_expect_tx(mb, P.step_bytes);
                bulk_g2s(my_ring + p_stage * P.stage_stride, p_ptr, P.step_bytes, mb);
            }
            if (++p_stage == nstage) p_stage = 0;
            p_ptr += P.step_bytes;
            if (++p_u < p_u1 && ++p_step == nsteps) {  // next (tile, matrix)
                p_step = 0;
                if (NMAT == 2 && p_mat == 0) {
                    p_mat = 1;
                } else {
                    p_mat = 0;
                    p_li++;
                }
                p_ptr = p_base(p_li, p_mat);
            }
        }
    };

    for (int i = tid; i < RED_FLOATS; i += THREADS) red[i] = 0.f;
    SLAI_TRACE_POINT(1)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    SLAI_TRACE_POINT(2)
    // The activation vector's loads go out first; the ring fill follows them into the memory system.
    const float inv_scale = stage_vector<PRO, F::SV_GRAN>(P, S, stat, Kp, [&]() {
        for (int s = 0; s < nstage; s++) issue();
    });
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    SLAI_TRACE_POINT(3)

    int c_stage = 0;
    uint32_t c_phase = 0;
    bool alive = true;
    for (int wv = 0; wv < n_waves; wv++) {
        int u0, u1;
        wave_range(wv, u0, u1);
        int u = u0;
        while (u < u1) {
            // one run of consecutive units inside the same (tile, matrix)
            const int li = u / upi, rem = u - li * upi;
            const int mat = NMAT == 2 ? rem / nsteps : 0;
            int step = rem - mat * nsteps;
            const int run_end = min(u1, u + (nsteps - step));
            float accA = 0.f, accB = 0.f;
            for (; u < run_end; u++, step++) {
                if (alive) alive = mbar_wait(my_mbar + 8 * c_stage, c_phase, P.err_flag);
                F::compute(my_ring + c_stage * P.stage_stride, step, L, S, accA, accB);
                __syncwarp();
                if (L.lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue();  // refill the stage just consumed
                if (++c_stage == nstage) {
                    c_stage = 0;
                    c_phase ^= 1;
                }
            }
            accA += __shfl_xor_sync(0xffffffffu, accA, 1);
            accA += __shfl_xor_sync(0xffffffffu, accA, 2);
            accB += __shfl_xor_sync(0xffffffffu, accB, 1);
            accB += __shfl_xor_sync(0xffffffffu, accB, 2);
            if (L.t == 0) {  // a warp has at most one run per (tile, matrix): plain stores
                float* dst = red + ((li * WARPS + warp) * NMAT + mat) * 16;
                dst[L.g] = accA;
                dst[L.g + 8] = accB;
            }
        }
        SLAI_TRACE_POINT(4)
        __syncthreads();
        SLAI_TRACE_POINT(5)
        // Epilogue of the wave: thread (li, r) adds the 16 partials of its row in warp order.
        const int items = min(WAVE, n_local - wv * WAVE);
        if (tid < items * 16) {
            const int li = tid >> 4, r = tid & 15;
            const int item = i0 + wv * WAVE + li;
            float val[NMAT];
#pragma unroll
            for (int mat = 0; mat < NMAT; mat++) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; w++) s += red[((li * WARPS + w) * NMAT + mat) * 16 + r];
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
                // rows 2i, 2i+1 of a tile sit in neighbouring lanes of the same half-warp
                const float other = __shfl_xor_sync(__activemask(), y, 1);
                if (P.rope && sg.role < 2) {
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
        SLAI_TRACE_POINT(6)
        if (wv + 1 < n_waves) {  // the partial buffer is reused by the next wave
            __syncthreads();
            for (int i = tid; i < RED_FLOATS; i += THREADS) red[i] = 0.f;
            __syncthreads();
        }
    }
}

// Dense f32 matrix (GpuQuantMatrix::F32): one warp per row.
__global__ void gemv_f32_kernel(float* out, const float* w, const float* v, int M, int K) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= M) return;
    const float* wr = w + (size_t)row * K;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(wr[k], v[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) out[row] = acc;
}

template <class F, int NMAT, int PRO, int EPI>
int launch_inst(slai_ctx* ctx, const GemvParams& P, int grid, size_t smem, bool pdl) {
    auto kern = gemv_kernel<F, NMAT, PRO, EPI>;
    static bool attr_done = false;  // per instantiation
    if (!attr_done) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
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

template <class F>
int launch_fmt(slai_ctx* ctx, const GemvParams& P, const GemvLaunch& L, int grid, size_t smem_fixed, size_t per_stage) {
    const bool pdl = L.pdl;
    // the partial-sum buffer of the dual (gate/up) kernel is twice as large
    const bool dual = L.epi == EPI_SILU;
    const size_t red_bytes = (size_t)WAVE * WARPS * (dual ? 2 : 1) * 16 * 4;
    const size_t fixed = smem_fixed + red_bytes;
    GemvParams Q = P;
    int nstage = (int)((SMEM_LIMIT - fixed) / per_stage);
    if (nstage > 6) nstage = 6;
    static int stage_env = -1;
    if (stage_env < 0) {
        const char* e = getenv("SLAI_GEMV_STAGES");
        stage_env = e ? atoi(e) : 0;
    }
    if (stage_env >= 2 && stage_env <= nstage) nstage = stage_env;
    SLAI_REQUIRE(ctx, nstage >= 2, SLAI_ERR_SHAPE, "gemv: K=%d does not fit in shared memory", P.K);
    Q.nstage = nstage;
    const size_t smem = fixed + (size_t)nstage * per_stage;
#define GO(NMAT, PRO, EPI) return launch_inst<F, NMAT, PRO, EPI>(ctx, Q, grid, smem, pdl)
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
        SLAI_CHECK_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_f32_kernel, L.out, (const float*)L.seg[0].w, L.v, M, K));
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
        SLAI_REQUIRE(ctx, ((uintptr_t)L.seg[s].w & 15) == 0, SLAI_ERR_INVALID_ARG, "gemv: matrix data must be 16-byte aligned");
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
    P.nsteps = (int)layout::num_steps(L.fmt, K);
    P.step_bytes = layout::step_bytes(L.fmt);
    P.stage_stride = (P.step_bytes + 127) & ~127;
    P.v = L.v; P.out = L.out; P.norm_w = L.norm_w; P.norm_b = L.norm_b; P.eps = L.eps;
    P.resid = L.resid; P.rope = L.rope; P.rope_theta = L.rope_theta; P.head_size = L.head_size;
    P.d_pos = L.d_pos; P.kcache = L.kcache; P.vcache = L.vcache; P.kv_f16 = (L.kv_dtype == SLAI_KV_F16);
    P.kv_pos_stride = L.kv_pos_stride; P.kv_head_stride = L.kv_head_stride;
    P.err_flag = ctx->d_counters + 3000;
#ifdef SLAI_TRACE
    P.trace = reinterpret_cast<unsigned long long*>(ctx->d_scratch);  // the debug driver sizes the scratch first
#endif

    const int Kp = (K + 255) & ~255;
    const int sv_gran = (L.fmt == SLAI_FMT_Q4_K || L.fmt == SLAI_FMT_Q5_K) ? 32 : L.fmt == SLAI_FMT_Q6_K ? 16 : 0;
    const size_t sv_bytes = sv_gran ? (size_t)(Kp / sv_gran) * 16 : 0;
    // everything except the partial-sum buffer and the ring
    const size_t fixed = (size_t)4 * (Kp + 32) + sv_bytes + 64 * 4 + WARPS * MAX_STAGES * 8 + 128;
    const size_t per_stage = (size_t)WARPS * P.stage_stride;
    int grid = P.n_items < ctx->sm_count ? P.n_items : ctx->sm_count;

    switch (L.fmt) {
        case SLAI_FMT_Q4_K: return launch_fmt<Q4K>(ctx, P, L, grid, fixed, per_stage);
        case SLAI_FMT_Q5_K: return launch_fmt<Q5K>(ctx, P, L, grid, fixed, per_stage);
        case SLAI_FMT_Q6_K: return launch_fmt<Q6K>(ctx, P, L, grid, fixed, per_stage);
        case SLAI_FMT_Q8_0: return launch_fmt<Q80>(ctx, P, L, grid, fixed, per_stage);
    }
    return slai_set_error(ctx, SLAI_ERR_UNSUPPORTED_FORMAT, "gemv: format %d has no kernel", L.fmt);
}
