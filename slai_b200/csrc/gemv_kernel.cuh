// Device side of the dequant-GEMV: shared by the stand-alone GEMV kernel (gemv.cu) and the persistent
// decode kernel that runs all layers of a token in one launch (decode.cu).
//
// Shape.  One persistent block of 16 warps per SM.  The weights are stored tile-major (layout.cuh): the packed
// data of 16 rows x one K step is one contiguous block.  Work is divided in two levels so that every SM and
// every warp gets the same amount (+-1 block) whatever the matrix shape: the 16-row tiles are dealt out in
// contiguous, equal runs to the thread blocks; inside a block of threads the run's sequence of
// (tile, matrix, K-step) units is cut into 16 equal contiguous pieces, one per warp.  A warp's piece may cover
// the end of one tile and the start of the next; its partial row sums go to shared memory, and after a barrier
// the 16 partials of every row are added in warp order (deterministic) and the epilogue runs.
//
// Data movement.  Every warp owns a private ring of shared-memory stages; one lane issues a bulk asynchronous
// copy (cp.async.bulk, completion counted on an mbarrier) per block, always NSTAGE blocks ahead of the block
// being consumed.  The producer walks a *program*: a list of GEMV phases.  For the stand-alone kernel the
// program has one entry; in the persistent decode kernel it lists every GEMV of every layer, so the ring keeps
// streaming the next phase's weights while the block of threads waits at the grid barrier between phases.
//
// Arithmetic.  Packed quants, four per register, go to the integer tensor-core MMA (mma.sync.m16n8k32 s8)
// against base-128 digit planes of the activation vector, staged once per phase in shared memory
// (gemv_frag.cuh); block scales are applied to the per-sub-block integer sums.
//
// Every mbarrier wait is bounded; on expiry the warp raises the error flag and stops waiting.
#pragma once
#include "common.cuh"
#include "gemv_frag.cuh"
#include "gemv_formats.cuh"
#include "layout.cuh"

namespace gemvk {

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
constexpr int RED_FLOATS = WAVE * WARPS * 2 * 16;  // partial sums (sized for the two-matrix gate/up phase)

struct GemvParams {
    GemvSeg seg[3];
    int nseg;
    int nmat;        // 2: gate/up pair (segments 0 and 1 processed tile by tile together), else 1
    int K;
    int n_items;     // 16-row tiles (nmat == 2: tiles of seg[0])
    int nsteps;      // tile-step blocks per tile
    int nstage;      // ring depth per warp
    int step_bytes;  // bytes of a tile-step block
    int stage_stride;
    int dig_region;  // bytes reserved at the start of shared memory for the staged vector (digits + sums)
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
// The vector is read once (L2 loads: inside the persistent kernel it was written by other SMs during the same
// launch, so L1 must not be trusted) and kept in registers between the passes when K <= 12288.
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
            xr[r] = i < n4 ? __ldcg(v4 + i) : zero4;
        }
    }
    after_loads();  // the vector's loads are in flight ahead of whatever this issues
    // element group of register slot r (CACHED) or of loop round r (not CACHED)
#define SLAI_STAGE_LOOP(...)                                                            \
    if (CACHED) {                                                                       \
        _Pragma("unroll") for (int r = 0; r < STAGE_REGS; r++) {                        \
            const int i = tid + r * THREADS;                                            \
            float4 x = xr[r];                                                           \
            __VA_ARGS__                                                                 \
        }                                                                               \
    } else {                                                                            \
        for (int i = tid; i < np4; i += THREADS) {                                      \
            float4 x = i < n4 ? __ldcg(v4 + i) : zero4;                                 \
            __VA_ARGS__                                                                 \
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
// Per-warp ring state and the producer that walks a program of GEMV phases.
// ---------------------------------------------------------------------------------------------
struct Ring {
    uint32_t mbar, ring;      // shared-space addresses of this warp's barriers and stages
    int nstage;
    uint32_t stage_stride, step_bytes;
    int c_stage;
    uint32_t c_phase;
    bool alive;
    unsigned int* err_flag;
    // producer
    const GemvParams* prog;
    int n_prog, p_idx;
    int i0, n_local, n_waves, upi, nsteps, nmat;  // geometry of program entry p_idx for this block of threads
    int p_wave, p_u, p_u1, p_li, p_mat, p_step, p_stage;
    const uint8_t* p_ptr;
};

// Shared-memory layout: [staged vector: dig_region bytes][red RED_FLOATS f32][stat 64 f32][mbar][ring]
__device__ __forceinline__ uint32_t smem_fixed_bytes(int dig_region) { return (uint32_t)dig_region + RED_FLOATS * 4 + 64 * 4; }

// this warp's unit range inside wave `wv` of a phase with `n_local` tiles of `upi` units
__device__ __forceinline__ void wave_range(int n_local, int upi, int wv, int warp, int& u0, int& u1) {
    const int items = min(WAVE, n_local - wv * WAVE);
    const int U = items * upi;
    u0 = (U * warp) / WARPS;
    u1 = (U * (warp + 1)) / WARPS;
}

__device__ __forceinline__ const uint8_t* prod_base(const Ring& R, int li, int mat) {
    const GemvParams& P = R.prog[R.p_idx];
    const int item = R.i0 + R.p_wave * WAVE + li;
    const int sidx = R.nmat == 2 ? mat : seg_of_tile(P, item);
    const GemvSeg& sg = P.seg[sidx];
    const int tile = R.nmat == 2 ? item : item - sg.tile0;
    return sg.w + (size_t)tile * sg.tile_bytes;
}
__device__ __forceinline__ void prod_seek(Ring& R) {  // divisions only here (once per wave)
    if (R.p_u < R.p_u1) {
        R.p_li = R.p_u / R.upi;
        const int rem = R.p_u - R.p_li * R.upi;
        R.p_mat = R.nmat == 2 ? rem / R.nsteps : 0;
        R.p_step = rem - R.p_mat * R.nsteps;
        R.p_ptr = prod_base(R, R.p_li, R.p_mat) + (size_t)R.p_step * R.step_bytes;
    }
}
__device__ __forceinline__ void prod_enter(Ring& R, int warp) {  // load the geometry of program entry p_idx
    if (R.p_idx >= R.n_prog) return;
    const GemvParams& P = R.prog[R.p_idx];
    R.nsteps = P.nsteps;
    R.nmat = P.nmat;
    R.upi = P.nsteps * P.nmat;
    R.i0 = (int)(((long long)P.n_items * blockIdx.x) / gridDim.x);
    const int i1 = (int)(((long long)P.n_items * (blockIdx.x + 1)) / gridDim.x);
    R.n_local = i1 - R.i0;
    R.n_waves = (R.n_local + WAVE - 1) / WAVE;
    R.p_wave = 0;
    R.p_u = R.p_u1 = 0;
    if (R.n_waves > 0) {
        wave_range(R.n_local, R.upi, 0, warp, R.p_u, R.p_u1);
        prod_seek(R);
    }
}
// Issue the copy of the next block of this warp's sequence (if any) into the next ring stage.
__device__ __forceinline__ void prod_issue(Ring& R, int lane, int warp) {
    while (R.p_idx < R.n_prog && (R.p_wave >= R.n_waves || R.p_u >= R.p_u1)) {  // skip exhausted waves / phases
        if (R.p_wave < R.n_waves && ++R.p_wave < R.n_waves) {
            wave_range(R.n_local, R.upi, R.p_wave, warp, R.p_u, R.p_u1);
            prod_seek(R);
        } else {
            R.p_idx++;
            prod_enter(R, warp);
        }
    }
    if (R.p_idx >= R.n_prog) return;
    if (lane == 0) {
        const uint32_t mb = R.mbar + 8 * R.p_stage;
        mbar_expect_tx(mb, R.step_bytes);
        bulk_g2s(R.ring + R.p_stage * R.stage_stride, R.p_ptr, R.step_bytes, mb);
    }
    if (++R.p_stage == R.nstage) R.p_stage = 0;
    R.p_ptr += R.step_bytes;
    if (++R.p_u < R.p_u1 && ++R.p_step == R.nsteps) {  // next (tile, matrix)
        R.p_step = 0;
        if (R.nmat == 2 && R.p_mat == 0) {
            R.p_mat = 1;
        } else {
            R.p_mat = 0;
            R.p_li++;
        }
        R.p_ptr = prod_base(R, R.p_li, R.p_mat);
    }
}

// Set up the ring of this warp for a program; P0 is the first entry (all entries share the ring geometry).
__device__ __forceinline__ void ring_init(Ring& R, const GemvParams* prog, int n_prog, unsigned char* smem_raw, int lane, int warp) {
    const GemvParams& P0 = prog[0];
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t mbar_base = base + smem_fixed_bytes(P0.dig_region);
    const uint32_t ring_base = (mbar_base + WARPS * MAX_STAGES * 8 + 127u) & ~127u;
    R.nstage = P0.nstage;
    R.stage_stride = P0.stage_stride;
    R.step_bytes = P0.step_bytes;
    R.mbar = mbar_base + warp * MAX_STAGES * 8;
    R.ring = ring_base + warp * R.nstage * R.stage_stride;
    R.c_stage = 0;
    R.c_phase = 0;
    R.alive = true;
    R.err_flag = P0.err_flag;
    R.prog = prog;
    R.n_prog = n_prog;
    R.p_idx = 0;
    R.p_stage = 0;
    R.p_ptr = nullptr;
    R.p_li = R.p_mat = R.p_step = 0;
    R.n_waves = 0;
    R.p_wave = 0;
    if (lane == 0) {
        for (int s = 0; s < R.nstage; s++) mbar_init(R.mbar + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    prod_enter(R, warp);
}

// ---------------------------------------------------------------------------------------------
// One GEMV phase (consumer side).  `first` : this is the first phase of the launch, whose ring fill has not
// been issued yet (it is issued right behind the activation loads).
// ---------------------------------------------------------------------------------------------
template <class F, int NMAT, int PRO, int EPI>
__device__ void gemv_phase(const GemvParams& P, Ring& R, unsigned char* smem_raw, bool first) {
    const int K = P.K;
    const int Kp = (K + 255) & ~255;
    constexpr int SV_BYTES_PER_256 = F::SV_GRAN > 0 ? 256 / F::SV_GRAN * 16 : 0;
    Smem S;
    S.dig = (uint32_t)__cvta_generic_to_shared(smem_raw);
    S.plane = Kp + 32;  // planes 32 bytes apart modulo 128: the four digit columns of a sub-block hit different banks
    S.sv = S.dig + 4 * S.plane;
    float* red = reinterpret_cast<float*>(smem_raw + P.dig_region);
    float* stat = red + RED_FLOATS;
    (void)SV_BYTES_PER_256;

    const int tid = threadIdx.x, warp = tid >> 5;
    LaneCtx L;
    lane_init(L, tid & 31, S);

    const int nsteps = P.nsteps;
    const int upi = nsteps * NMAT;
    const int i0 = (int)(((long long)P.n_items * blockIdx.x) / gridDim.x);
    const int i1 = (int)(((long long)P.n_items * (blockIdx.x + 1)) / gridDim.x);
    const int n_local = i1 - i0;
    const int n_waves = (n_local + WAVE - 1) / WAVE;

    for (int i = tid; i < WAVE * WARPS * NMAT * 16; i += THREADS) red[i] = 0.f;
    SLAI_TRACE_POINT(2)
    // The activation vector's loads go out first; the first ring fill follows them into the memory system.
    const float inv_scale = stage_vector<PRO, F::SV_GRAN>(P, S, stat, Kp, [&]() {
        if (first)
            for (int s = 0; s < R.nstage; s++) prod_issue(R, L.lane, warp);
    });
    SLAI_TRACE_POINT(3)

    for (int wv = 0; wv < n_waves; wv++) {
        int u, u1;
        wave_range(n_local, upi, wv, warp, u, u1);
        while (u < u1) {
            // one run of consecutive units inside the same (tile, matrix)
            const int li = u / upi, rem = u - li * upi;
            const int mat = NMAT == 2 ? rem / nsteps : 0;
            int step = rem - mat * nsteps;
            const int run_end = min(u1, u + (nsteps - step));
            float accA = 0.f, accB = 0.f;
            for (; u < run_end; u++, step++) {
                if (R.alive) R.alive = mbar_wait(R.mbar + 8 * R.c_stage, R.c_phase, R.err_flag);
                F::compute(R.ring + R.c_stage * R.stage_stride, step, L, S, accA, accB);
                __syncwarp();
                if (L.lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                prod_issue(R, L.lane, warp);  // refill the stage just consumed
                if (++R.c_stage == R.nstage) {
                    R.c_stage = 0;
                    R.c_phase ^= 1;
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
                if (valid) P.out[orow] = __ldcg(P.resid + orow) + (val[0] + bias);
            } else if (EPI == EPI_SILU) {
                if (valid) {
                    const float gt = val[0], up = val[NMAT - 1];
                    P.out[orow] = up * (gt / (1.0f + expf(-gt)));
                }
            } else if (EPI == EPI_GELU) {
                if (valid) P.out[orow] = gelu_ref(val[0] + bias);
            } else if (EPI == EPI_QKV) {
                float y = val[0] + bias;
                const int pos = __ldcg(P.d_pos);
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
            for (int i = tid; i < WAVE * WARPS * NMAT * 16; i += THREADS) red[i] = 0.f;
            __syncthreads();
        }
    }
}

}  // namespace gemvk

// gemv.cu: validate a launch description and turn it into kernel parameters (dig_region / nstage 0 = size them
// for this launch alone).
int gemv_fill_params(slai_ctx* ctx, const GemvLaunch& L, size_t dig_region, int nstage, gemvk::GemvParams& P, size_t* smem_out,
                     int* grid_out);
