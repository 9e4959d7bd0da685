// Device side of the dequant-GEMV kernel (gemv.cu).
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
// being consumed.  The ring starts filling before the wait for the predecessor (programmatic dependent launch).
//
// Arithmetic.  Packed quants, four per register, go to the integer tensor-core MMA (mma.sync.m16n8k32 s8)
// against base-256 digit planes of the activation vector, staged once per phase in shared memory
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

// Build-time knobs of the measurements behind the shipped shape (SLAI_NVCC_EXTRA="-D..." python -m slai_b200.build):
// warps per block, and the minimum number of blocks per SM the compiler sizes the registers for (2 = 64 registers per
// thread at 16 warps, so that the next kernel's blocks are resident while this one runs).  16 warps / 1 block measured
// fastest; 8 warps and 2 blocks per SM both lose more in the main loop than the early residency gains.
#ifndef SLAI_GEMV_WARPS
#define SLAI_GEMV_WARPS 16
#endif
constexpr int WARPS = SLAI_GEMV_WARPS;
#ifndef SLAI_GEMV_MINB
#define SLAI_GEMV_MINB 1
#endif
constexpr int THREADS = 32 * WARPS;
constexpr int MAX_STAGES = 8;  // ring depth limit (host side)
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
    int items_base, items_rem;  // items per block of threads: base each, one more for the first `rem`
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
    const float* rope_cs;  // (cos, sin) pairs of the current position, or null
    int head_size;
    const int* d_pos;
    int pos1;        // position + 1 when the caller already knows it (0: read d_pos)
    void* kcache;
    void* vcache;
    float* k_out;    // EPI_QKV: k rows as f32 instead of the cache (null: cache)
    int kv_f16;
    long long kv_pos_stride, kv_head_stride;
    unsigned int* err_flag;
    unsigned int wait_limit;  // rounds a bounded wait polls before it raises err_flag and goes on
    int pdl;  // launched with programmatic stream serialization (2: trigger the dependent launch at the start)
    const char* pf_ptr;  // memory the next kernel reads first: prefetched into L2 by one block (pf_lines x 128 bytes)
    int pf_lines;
    PrefetchPlan ahead;  // weights of a later kernel, pulled into L2 by all blocks at the start
    // tensor-parallel exchange over peer memory (xr == 0: unused)
    int xr, xrank;                       // ranks in the group, this rank
    uint2* xo_slot[XCHG_MAX_RANKS];      // EPI_XCHG: this rank's slot of the outgoing exchange in every rank's region
    unsigned int xo_idx1, xi_idx1, x_per_token;  // exchange index + 1 inside the token (out / in), exchanges per token
    const uint2* xi_slots;               // incoming exchange in this rank's region: [ranks][XCHG_MAX_DIM] (null: read `v`)
    const unsigned int* x_tokseq;        // device scalar: tokens decoded so far
    float* xsum_out;                     // the summed incoming vector is left here (for the residual of the next exchange)
    uint2* xl_sum;                       // non-null: two-level sum -- each block sums a slice over the ranks into this local
                                         // tagged buffer, then every block reads the whole sum from it
#ifdef SLAI_TRACE
    unsigned long long* trace;   // trace build only: per block of threads TRACE_POINTS globaltimer stamps
    unsigned long long* tl;      // trace build only: the context's launch timeline
#endif
};

#ifdef SLAI_TRACE
#define SLAI_TRACE_POINT(k) \
    if (threadIdx.x == 0 && P.trace) P.trace[blockIdx.x * TRACE_POINTS + (k)] = slai_globaltimer();
#else
#define SLAI_TRACE_POINT(k)
#endif

// ---- mbarrier / bulk copy -------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
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

// ---- tensor-parallel exchange over peer memory ----------------------------------------------------------------
// Every element travels as one 8-byte store (value, sequence tag).  The tag of exchange `idx1` of the current token
// only ever grows from exchange to exchange, so "tag == seq" means "this rank's partial of this exchange has
// arrived": no flags, no fences, one NVLink store latency.
__device__ __forceinline__ unsigned int xchg_seq(const GemvParams& P, unsigned int idx1) {
    return __ldcg(P.x_tokseq) * P.x_per_token + idx1;
}
// Sum over the ranks, in rank order, of element group i (four floats) of the incoming exchange; identical on every
// rank.  Polls (bounded) until all four tags of every rank match; on expiry the error flag is raised and the
// kernel goes on with whatever is there.
__device__ __forceinline__ void xchg_load(const uint4* src, uint4& a, uint4& b) {
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(src + 1) : "memory");
}
__device__ __forceinline__ float4 xchg_gather(const GemvParams& P, int i, unsigned int seq) {
    const uint4* src = reinterpret_cast<const uint4*>(P.xi_slots + 4 * (size_t)i);
    constexpr size_t RANK_STRIDE = (size_t)XCHG_MAX_DIM * sizeof(uint2) / sizeof(uint4);
    uint4 a[XCHG_MAX_RANKS], b[XCHG_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < XCHG_MAX_RANKS; r++)  // all ranks' loads go out together: one trip when everything has arrived
        if (r < P.xr) xchg_load(src + r * RANK_STRIDE, a[r], b[r]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < XCHG_MAX_RANKS; r++)
        if (r < P.xr) {
            for (int it = 0; !(a[r].y == seq && a[r].w == seq && b[r].y == seq && b[r].w == seq); it++) {
                if ((unsigned int)it > P.wait_limit) {
                    atomicExch(P.err_flag, 3u);
                    break;
                }
                if (it > 16) __nanosleep(100);
                xchg_load(src + r * RANK_STRIDE, a[r], b[r]);
            }
            acc.x += __uint_as_float(a[r].x); acc.y += __uint_as_float(a[r].z);
            acc.z += __uint_as_float(b[r].x); acc.w += __uint_as_float(b[r].z);
        }
    return acc;
}

// Element group i of the two-level sum, from this GPU's own tagged buffer (written by the block that owns the slice).
__device__ __forceinline__ float4 xchg_local(const GemvParams& P, int i, unsigned int seq) {
    const uint4* src = reinterpret_cast<const uint4*>(P.xl_sum + 4 * (size_t)i);
    uint4 a, b;
    xchg_load(src, a, b);
    for (int it = 0; !(a.y == seq && a.w == seq && b.y == seq && b.w == seq); it++) {
        if ((unsigned int)it > P.wait_limit) {
            atomicExch(P.err_flag, 3u);
            break;
        }
        if (it > 16) __nanosleep(100);
        xchg_load(src, a, b);
    }
    return make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
}

// Stage the activation vector: optional normalisation, power-of-two scaling so that max|v| lands in
// [2^25, 2^26), rounding to integers, split into four base-256 digit planes (gemv_frag.cuh), and per-sub-block
// digit sums (for the `- dmin*m * sum(v)` term of Q4_K / Q5_K and the -32 offset of Q6_K).  Returns 1/scale.
// The vector is read once (L2 loads: it was written by the kernel launched just before, on other SMs) and kept in
// registers between the passes when K <= 12288 (the digit pass is unrolled over the register copy, so that its
// rounds overlap); longer vectors are read again in each pass, four loads in flight per thread.
// XIN: the vector is the sum over ranks of an incoming tensor-parallel exchange (K <= 24576 so that it stays in
// registers); block 0 also writes the sum to P.xsum_out.
template <int SV_GRAN, bool HAS_LN, bool XIN>
__device__ __forceinline__ float stage_vector(const int PRO_ARG, const GemvParams& P, const Smem& S, float* stat, int Kp) {
    const int PRO = (!HAS_LN && PRO_ARG == PRO_LN) ? PRO_RMS : PRO_ARG;  // LayerNorm code only where it can occur
    const int K = P.K;
    const int tid = threadIdx.x;
    const float4* v4 = reinterpret_cast<const float4*>(P.v);
    const float4* w4p = reinterpret_cast<const float4*>(P.norm_w);
    const float4* b4p = reinterpret_cast<const float4*>(P.norm_b);
    const int n4 = K >> 2, np4 = Kp >> 2;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool cached = np4 <= STAGE_REGS * THREADS;
    float4 xr[STAGE_REGS];
    const unsigned int xseq = XIN ? xchg_seq(P, P.xi_idx1) : 0u;
    if (XIN && P.xl_sum) {
        // Two-level sum (many ranks): reading every rank's partial in every block would move ranks x 64 KB through L2
        // per block.  Each block sums only its slice over the ranks and publishes it, tagged, in a local buffer.
        const int g0 = (int)(((long long)n4 * blockIdx.x) / gridDim.x), g1 = (int)(((long long)n4 * (blockIdx.x + 1)) / gridDim.x);
        for (int i = g0 + tid; i < g1; i += THREADS) {
            const float4 sum = xchg_gather(P, i, xseq);
            reinterpret_cast<float4*>(P.xsum_out)[i] = sum;
            uint4* dst = reinterpret_cast<uint4*>(P.xl_sum + 4 * (size_t)i);
            dst[0] = make_uint4(__float_as_uint(sum.x), xseq, __float_as_uint(sum.y), xseq);
            dst[1] = make_uint4(__float_as_uint(sum.z), xseq, __float_as_uint(sum.w), xseq);
        }
    }
#pragma unroll
    for (int r = 0; r < STAGE_REGS; r++) {
        const int i = tid + r * THREADS;
        if (XIN) {
            if (P.xl_sum) {
                xr[r] = i < n4 ? xchg_local(P, i, xseq) : zero4;
            } else {
                xr[r] = i < n4 ? xchg_gather(P, i, xseq) : zero4;
                if (blockIdx.x == 0 && i < n4) reinterpret_cast<float4*>(P.xsum_out)[i] = xr[r];
            }
        } else {
            xr[r] = (cached && i < n4) ? __ldcg(v4 + i) : zero4;
        }
    }
    float mul = 1.f, sub = 0.f;
    float sum = 0.f, mx = 0.f;
    if (HAS_LN && PRO == PRO_LN) {
        if (cached) {
#pragma unroll
            for (int r = 0; r < STAGE_REGS; r++) sum += (xr[r].x + xr[r].y) + (xr[r].z + xr[r].w);
        } else {
#pragma unroll 1
            for (int i = tid; i < n4; i += THREADS) {
                const float4 x = __ldcg(v4 + i);
                sum += (x.x + x.y) + (x.z + x.w);
            }
        }
        block_sum_max(sum, mx, stat);
        sub = sum / (float)K;
        sum = 0.f;
    }
    auto stats = [&](float4 x, const float4& w) {
        if (PRO == PRO_NONE) {
            mx = fmaxf(mx, max4(x));
        } else {
            if (HAS_LN && PRO == PRO_LN) { x.x -= sub; x.y -= sub; x.z -= sub; x.w -= sub; }
            sum += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
            mx = fmaxf(mx, max4(make_float4(x.x * w.x, x.y * w.y, x.z * w.z, x.w * w.w)));
        }
    };
    float4 wr[STAGE_REGS];  // norm weights of the register copy: all requested before the first is used, kept for the digit pass
    if (cached) {
#pragma unroll
        for (int r = 0; r < STAGE_REGS; r++) {
            const int i = tid + r * THREADS;
            wr[r] = (PRO != PRO_NONE && i < n4) ? __ldg(w4p + i) : zero4;
        }
#pragma unroll
        for (int r = 0; r < STAGE_REGS; r++)
            if (tid + r * THREADS < n4) stats(xr[r], wr[r]);
    } else {
        // long vectors: four loads in flight per thread and round (one at a time would pay the L2 latency every round)
#pragma unroll 1
        for (int i0 = tid; i0 < n4; i0 += 4 * THREADS) {
            float4 xb[4], wb[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * THREADS;
                xb[u] = i < n4 ? __ldcg(v4 + i) : zero4;
                wb[u] = (PRO != PRO_NONE && i < n4) ? __ldg(w4p + i) : zero4;
            }
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (i0 + u * THREADS < n4) stats(xb[u], wb[u]);
        }
    }
    SLAI_TRACE_POINT(6)
    block_sum_max(sum, mx, stat);
    SLAI_TRACE_POINT(7)
    if (PRO != PRO_NONE) {
        mul = 1.0f / sqrtf(sum / (float)K + P.eps);
        mx *= mul;
        if (HAS_LN && PRO == PRO_LN && P.norm_b) {
            float mb = 0.f, dummy = 0.f;
#pragma unroll 1
            for (int i = tid; i < n4; i += THREADS) mb = fmaxf(mb, max4(__ldg(b4p + i)));
            block_sum_max(dummy, mb, stat);
            mx += mb;
        }
    }
    float scale = 1.f;
    if (mx > 0.f && mx < 3.0e38f) {
        int e = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 126;  // mx = f * 2^e with f in [0.5, 1) (normal numbers)
        if ((__float_as_uint(mx) >> 23) == 0u) e = -126;              // subnormal: scale as the smallest normal
        e = e < -90 ? -90 : e;
        scale = __uint_as_float((uint32_t)(127 + 26 - e) << 23);       // 2^(26 - e), exact
    }
    unsigned char* dig = reinterpret_cast<unsigned char*>(__cvta_shared_to_generic(S.dig));
    int4* sv = reinterpret_cast<int4*>(__cvta_shared_to_generic(S.sv));
    unsigned char* svb = reinterpret_cast<unsigned char*>(sv);  // Q4_K / Q5_K: byte table of the sums (gemv_formats.cuh)
    if (tid < ZERO_BYTES / 4) reinterpret_cast<uint32_t*>(__cvta_shared_to_generic(S.zero))[tid] = 0u;
    // One float4 (elements 4i .. 4i+3): normalise, round to integers, digits, sums.  np4 is a multiple of 64, so whole
    // warps take part in every call (the sums are reduced with shuffles).
    auto convert = [&](float4 x, const float4& w, const int i) {
        if (i < n4 && PRO != PRO_NONE) {
            if (HAS_LN && PRO == PRO_LN) { x.x -= sub; x.y -= sub; x.z -= sub; x.w -= sub; }
            x.x = (x.x * mul) * w.x; x.y = (x.y * mul) * w.y; x.z = (x.z * mul) * w.z; x.w = (x.w * mul) * w.w;
            if (HAS_LN && PRO == PRO_LN && P.norm_b) {
                const float4 b = __ldg(b4p + i);
                x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
            }
        }
        // four digits per element in one word (two instructions each), then a 4 x 4 byte transpose into plane words
        uint32_t pw[4];
        digit_planes(digits_word(__float2int_rn(x.x * scale)), digits_word(__float2int_rn(x.y * scale)),
                     digits_word(__float2int_rn(x.z * scale)), digits_word(__float2int_rn(x.w * scale)), pw);
#pragma unroll
        for (int q = 0; q < 4; q++) *reinterpret_cast<uint32_t*>(dig + (size_t)q * S.plane + 4 * i) = pw[q];
        if (SV_GRAN > 0) {
            constexpr int LANES = SV_GRAN > 0 ? SV_GRAN / 4 : 1;  // float4 groups per sub-block
            constexpr int BIAS = 512;                             // a float4's digit sum lies in [-512, 508]
            // two biased sums per word, so that a shuffle round serves two digit planes
            uint32_t s01 = (uint32_t)__dp4a((int)pw[0], 0x01010101, BIAS) | ((uint32_t)__dp4a((int)pw[1], 0x01010101, BIAS) << 16);
            uint32_t s23 = (uint32_t)__dp4a((int)pw[2], 0x01010101, BIAS) | ((uint32_t)__dp4a((int)pw[3], 0x01010101, BIAS) << 16);
#pragma unroll
            for (int o = 1; o < LANES; o <<= 1) {
                s01 += __shfl_xor_sync(0xffffffffu, s01, o);
                s23 += __shfl_xor_sync(0xffffffffu, s23, o);
            }
            if ((tid & (LANES - 1)) == 0) {
                const int sd[4] = {(int)(s01 & 0xFFFFu) - BIAS * LANES, (int)(s01 >> 16) - BIAS * LANES, (int)(s23 & 0xFFFFu) - BIAS * LANES,
                                   (int)(s23 >> 16) - BIAS * LANES};
                if (SV_GRAN == 32) {
                    // sub-block J = i / 8 of step J / 8: every sum (|sum| <= 4096) as two base-128 digits, one byte row per
                    // (digit plane, part); bytes 8..15 of the sub-block's own row index are the zero half of that row
                    const int J = i >> 3;
                    unsigned char* tab = svb + (J >> 3) * 128;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int hi = (sd[q] + 64) >> 7, lo = sd[q] - (hi << 7);
                        tab[(2 * q) * 16 + (J & 7)] = (unsigned char)hi;
                        tab[(2 * q + 1) * 16 + (J & 7)] = (unsigned char)lo;
                    }
                    *reinterpret_cast<uint2*>(tab + (J & 7) * 16 + 8) = make_uint2(0u, 0u);
                } else {
                    sv[i / LANES] = make_int4(sd[0], sd[1], sd[2], sd[3]);
                }
            }
        }
    };
    if (cached) {
#pragma unroll
        for (int r = 0; r < STAGE_REGS; r++)
            if (tid + r * THREADS < np4) convert(xr[r], wr[r], tid + r * THREADS);  // independent rounds: the compiler overlaps them
    } else {
#pragma unroll 1
        for (int i0 = tid; i0 < np4; i0 += 4 * THREADS) {
            float4 xb[4], wb[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * THREADS;
                xb[u] = i < n4 ? __ldcg(v4 + i) : zero4;
                wb[u] = (PRO != PRO_NONE && i < n4) ? __ldg(w4p + i) : zero4;
            }
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (i0 + u * THREADS < np4) convert(xb[u], wb[u], i0 + u * THREADS);
        }
    }
    SLAI_TRACE_POINT(8)
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
// Segment `s` by value through selects (a dynamically indexed copy of the parameter array would go to local memory).
__device__ __forceinline__ GemvSeg seg_pick(const GemvParams& P, int s) {
    GemvSeg r = P.seg[0];
    if (P.nseg > 1 && s == 1) r = P.seg[1];
    if (P.nseg > 2 && s == 2) r = P.seg[2];
    return r;
}

// First tile-step block of (item, matrix): items are 16-row tiles (of segment 0 and 1 together for the gate/up pair).
__device__ __forceinline__ const uint8_t* tile_ptr(const GemvParams& P, int item, int mat) {
    const int sidx = P.nmat == 2 ? mat : seg_of_tile(P, item);
    const uint8_t* w = P.seg[0].w;
    long long tb = P.seg[0].tile_bytes;
    int t0 = 0;
    if (sidx == 1) { w = P.seg[1].w; tb = P.seg[1].tile_bytes; t0 = P.seg[1].tile0; }
    if (sidx == 2) { w = P.seg[2].w; tb = P.seg[2].tile_bytes; t0 = P.seg[2].tile0; }
    const int tile = P.nmat == 2 ? item : item - t0;
    return w + (size_t)tile * tb;
}

// ---------------------------------------------------------------------------------------------
// Work split.  A block of threads owns `n_local` consecutive items starting at `i0`; they are processed in waves
// of WAVE items, and the wave's sequence of (item, matrix, step) units is cut into WARPS equal pieces.  A cursor
// walks one warp's piece run by run (a run = consecutive steps of one (item, matrix)); the consumer and the ring
// producer (which is `nstage` units ahead) each have one.  Division-free.
// ---------------------------------------------------------------------------------------------
struct Split {
    int i0, n_local, n_waves, upi, nsteps, nmat;
};
__device__ __forceinline__ Split make_split(const GemvParams& P) {
    Split s;
    const int b = (int)blockIdx.x;
    s.i0 = b * P.items_base + min(b, P.items_rem);
    s.n_local = P.items_base + (b < P.items_rem ? 1 : 0);
    s.n_waves = (s.n_local + WAVE - 1) / WAVE;
    s.nsteps = P.nsteps;
    s.nmat = P.nmat;
    s.upi = P.nsteps * P.nmat;
    return s;
}
struct Cursor {
    int wave, li, mat, step;
    int left;  // units of the piece not yet walked
};
// Position the cursor on this warp's piece of wave `c.wave`.
__device__ __forceinline__ void cursor_wave(Cursor& c, const Split& s, int warp) {
    const int items = min(WAVE, s.n_local - c.wave * WAVE);
    const int U = items * s.upi;
    const int u0 = (U * warp) / WARPS;
    c.left = (U * (warp + 1)) / WARPS - u0;
    int rem = u0;
    c.li = 0;
    while (rem >= s.upi) {  // at most WAVE rounds
        rem -= s.upi;
        c.li++;
    }
    c.mat = 0;
    if (rem >= s.nsteps) {  // only with two matrices per item
        rem -= s.nsteps;
        c.mat = 1;
    }
    c.step = rem;
}
// After the last step of a run: first step of the next (item, matrix).
__device__ __forceinline__ void cursor_next_run(Cursor& c, const Split& s) {
    c.step = 0;
    if (s.nmat == 2 && c.mat == 0) {
        c.mat = 1;
    } else {
        c.mat = 0;
        c.li++;
    }
}

// ---------------------------------------------------------------------------------------------
// Per-warp ring.  A stage is STRIDE bytes: one tile-step block and, in its last 8 bytes, the mbarrier its bulk copy
// completes on.  The warp that consumes a stage refills it at once with the block `nstage` units further down its
// sequence.  Stage size and barrier offset are compile-time constants of the format, and the request is one
// predicated instruction sequence (no divergent branch), so the common path is a handful of instructions; run and
// wave changes are off that path.
// ---------------------------------------------------------------------------------------------
template <class F>
struct RingGeom {
    static constexpr uint32_t STEP = F::STEP_BYTES;
    static constexpr uint32_t STRIDE = (STEP + 8 + 127) & ~127u;
    static constexpr uint32_t MBAR = STRIDE - 8;
};
struct Ring {
    uint32_t base, end;       // shared-space addresses of this warp's stages [base, end)
    uint32_t c_addr;          // stage consumed next
    uint32_t c_phase;
    uint32_t lane0;           // 1 in the lane that requests the copies
    unsigned int limit;       // polls a wait may take; 1 after a wait has expired (later waits give up at once)
    unsigned int* err_flag;
    // producer
    Cursor pc;
    int p_run;                // units left in the producer's run (<= 0: nothing more to request)
    const uint8_t* p_ptr;
};

// Shared-memory layout: [staged vector: dig_region bytes = zero page, digit planes, digit sums][red RED_FLOATS f32][stat 64 f32][ring]
__device__ __forceinline__ uint32_t smem_fixed_bytes(int dig_region) { return (uint32_t)dig_region + RED_FLOATS * 4 + 64 * 4; }

// Bounded wait for the phase `parity` of the barrier at `a`.  On expiry the error flag is raised and `limit` drops to
// one poll, so that the kernel still ends quickly.
__device__ __forceinline__ void ring_wait(uint32_t a, uint32_t parity, unsigned int& limit, unsigned int* err_flag) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .u32 n;\n\tmov.u32 n, 0;\n"
        "W:\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t@p bra D;\n\tadd.u32 n, n, 1;\n\tsetp.lt.u32 p, n, %3;\n\t@p bra W;\n\t"
        "mov.u32 %0, 0;\n\tbra E;\n"
        "D:\n\tmov.u32 %0, 1;\n"
        "E:\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity), "r"(limit)
        : "memory");
    if (!ok) {
        atomicExch(err_flag, 1u);
        limit = 1;
    }
}

template <class F>
__device__ __forceinline__ void prod_run(Ring& R, const GemvParams& P, const Split& sp) {
    R.p_run = min(R.pc.left, sp.nsteps - R.pc.step);
    R.pc.left -= R.p_run;
    R.p_ptr = tile_ptr(P, sp.i0 + R.pc.wave * WAVE + R.pc.li, R.pc.mat) + (size_t)R.pc.step * RingGeom<F>::STEP;
}
// First non-empty piece from wave `pc.wave` on.
template <class F>
__device__ __forceinline__ void prod_open(Ring& R, const GemvParams& P, const Split& sp, int warp) {
    R.p_run = 0;
    for (; R.pc.wave < sp.n_waves; R.pc.wave++) {
        cursor_wave(R.pc, sp, warp);
        if (R.pc.left > 0) {
            prod_run<F>(R, P, sp);
            return;
        }
    }
}
template <class F>
__device__ __forceinline__ void prod_advance(Ring& R, const GemvParams& P, const Split& sp, int warp) {
    if (R.pc.left > 0) {
        cursor_next_run(R.pc, sp);
        prod_run<F>(R, P, sp);
    } else {
        R.pc.wave++;
        prod_open<F>(R, P, sp, warp);
    }
}
// Request the next block of the warp's sequence (if any) into the stage at `stage` (which this warp has finished
// reading: the proxy fence orders those reads before the asynchronous write).
template <class F>
__device__ __forceinline__ void prod_step(Ring& R, const GemvParams& P, const Split& sp, uint32_t stage, int warp) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.gt.s32 p, %0, 0;\n\tsetp.ne.and.u32 p, %1, 0, p;\n\t"
        "@p fence.proxy.async.shared::cta;\n\t"
        "@p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%2+%5], %4;\n\t"
        "@p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%2], [%3], %4, [%2+%5];\n\t}"
        :
        : "r"(R.p_run), "r"(R.lane0), "r"(stage), "l"(R.p_ptr), "n"(RingGeom<F>::STEP), "n"(RingGeom<F>::MBAR)
        : "memory");
    R.p_ptr += RingGeom<F>::STEP;
    if (--R.p_run == 0) prod_advance<F>(R, P, sp, warp);
}

// Barriers of this warp's ring; nothing is requested yet.
template <class F>
__device__ __forceinline__ void ring_setup(Ring& R, const GemvParams& P, unsigned char* smem_raw, int lane, int warp) {
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t ring_base = (base + smem_fixed_bytes(P.dig_region) + 127u) & ~127u;
    R.base = ring_base + warp * P.nstage * RingGeom<F>::STRIDE;
    R.end = R.base + P.nstage * RingGeom<F>::STRIDE;
    R.c_addr = R.base;
    R.c_phase = 0;
    R.lane0 = lane == 0 ? 1u : 0u;
    R.limit = P.wait_limit;
    R.err_flag = P.err_flag;
    R.p_run = 0;
    R.p_ptr = nullptr;
    if (lane == 0) {
        for (uint32_t a = R.base; a < R.end; a += RingGeom<F>::STRIDE) mbar_init(a + RingGeom<F>::MBAR, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
}
// Start the stream: the first `nstage` blocks of the warp's sequence.
template <class F>
__device__ __forceinline__ void ring_fill(Ring& R, const GemvParams& P, const Split& sp, int warp) {
    R.pc.wave = 0;
    prod_open<F>(R, P, sp, warp);
#pragma unroll 1
    for (uint32_t a = R.base; a < R.end; a += RingGeom<F>::STRIDE) prod_step<F>(R, P, sp, a, warp);
}

// ---------------------------------------------------------------------------------------------
// The GEMV after the predecessor's results are visible: stage the vector, main loop, epilogue.
// ---------------------------------------------------------------------------------------------
template <class F, int NMAT, int PRO, int EPI, bool XIN>
__device__ __forceinline__ void gemv_body(const GemvParams& P, Ring& R, const Split& sp, unsigned char* smem_raw) {
#define SLAI_EPI_IS(x) (EPI == (x))
    const int K = P.K;
    const int Kp = (K + 255) & ~255;
    Smem S;
    S.zero = (uint32_t)__cvta_generic_to_shared(smem_raw);
    S.dig = S.zero + ZERO_BYTES;
    S.plane = Kp + 32;  // planes 32 bytes apart modulo 128: the four digit columns of a sub-block hit different banks
    S.sv = S.dig + 4 * S.plane;
    float* red = reinterpret_cast<float*>(smem_raw + P.dig_region);
    float* stat = red + RED_FLOATS;

    const int tid = threadIdx.x, warp = tid >> 5;
    LaneCtx L;
    lane_init<F>(L, tid & 31, S);

    SLAI_TRACE_POINT(5)
    const float inv_scale = stage_vector<F::SV_GRAN, PRO == PRO_LN, XIN>(PRO, P, S, stat, Kp);
    SLAI_TRACE_POINT(9)

    Cursor c;
    for (c.wave = 0; c.wave < sp.n_waves; c.wave++) {
        // Epilogue operands that do not depend on the products (residual, bias, RoPE cos / sin) are requested now and
        // used after the loop: their L2 latency hides behind the wave instead of standing at the end of the kernel.
        float e_resid = 0.f, e_bias = 0.f, e_cs = 1.f, e_sn = 0.f;
        {
            const int items = min(WAVE, sp.n_local - c.wave * WAVE);
            if (tid < items * 16) {
                const int li = tid >> 4, r = tid & 15;
                const int item = sp.i0 + c.wave * WAVE + li;
                const GemvSeg sg = seg_pick(P, NMAT == 2 ? 0 : seg_of_tile(P, item));
                const int row_in_seg = (NMAT == 2 ? item : item - sg.tile0) * 16 + r;
                const bool valid = row_in_seg < sg.rows;
                const int orow = sg.out_off + row_in_seg;
                if (sg.bias && valid) e_bias = sg.bias[row_in_seg];
                if ((SLAI_EPI_IS(EPI_RESID) || (SLAI_EPI_IS(EPI_XCHG) && P.xrank == 0)) && valid) e_resid = __ldcg(P.resid + orow);
                if (SLAI_EPI_IS(EPI_QKV) && P.rope && sg.role < 2 && P.rope_cs) {
                    const int hd = (row_in_seg & ~1) % P.head_size;
                    e_cs = __ldcg(P.rope_cs + hd);
                    e_sn = __ldcg(P.rope_cs + hd + 1);
                }
            }
        }
        cursor_wave(c, sp, warp);
        while (c.left > 0) {
            const int run = min(c.left, sp.nsteps - c.step);
            float accA = 0.f, accB = 0.f;
            int step = c.step;
#pragma unroll 1
            for (int i = run; i > 0; i--, step++) {
                ring_wait(R.c_addr + RingGeom<F>::MBAR, R.c_phase, R.limit, R.err_flag);
                F::compute(R.c_addr, step, L, S, accA, accB);
                __syncwarp();
                prod_step<F>(R, P, sp, R.c_addr, warp);  // refill the stage just consumed
                R.c_addr += RingGeom<F>::STRIDE;
                if (R.c_addr == R.end) {
                    R.c_addr = R.base;
                    R.c_phase ^= 1;
                }
            }
            c.left -= run;
            accA += __shfl_xor_sync(0xffffffffu, accA, 1);
            accA += __shfl_xor_sync(0xffffffffu, accA, 2);
            accB += __shfl_xor_sync(0xffffffffu, accB, 1);
            accB += __shfl_xor_sync(0xffffffffu, accB, 2);
            if (L.t == 0) {  // a warp has at most one run per (item, matrix): plain stores
                float* dst = red + ((c.li * WARPS + warp) * NMAT + c.mat) * 16;
                dst[L.g] = accA;
                dst[L.g + 8] = accB;
            }
            cursor_next_run(c, sp);
        }
        const int wv = c.wave, n_waves = sp.n_waves, n_local = sp.n_local, i0 = sp.i0;
        SLAI_TRACE_POINT(10)
        __syncthreads();
        SLAI_TRACE_POINT(11)
        // Epilogue of the wave: thread (li, r) adds the 16 partials of its row in warp order.
        const int items = min(WAVE, n_local - wv * WAVE);
        if (tid < items * 16) {
            const int li = tid >> 4, r = tid & 15;
            const int item = i0 + wv * WAVE + li;
            float val[2] = {0.f, 0.f};
#pragma unroll
            for (int mat = 0; mat < 2; mat++)
                if (mat < NMAT) {
                    float s = 0.f;
#pragma unroll
                    for (int w = 0; w < WARPS; w++) s += red[((li * WARPS + w) * NMAT + mat) * 16 + r];
                    val[mat] = s * inv_scale;
                }
            const int sidx = NMAT == 2 ? 0 : seg_of_tile(P, item);
            const GemvSeg sg = seg_pick(P, sidx);
            const int row_in_seg = (NMAT == 2 ? item : item - sg.tile0) * 16 + r;
            const bool valid = row_in_seg < sg.rows;
            const int orow = sg.out_off + row_in_seg;
            const float bias = e_bias;
            if (SLAI_EPI_IS(EPI_STORE)) {
                if (valid) P.out[orow] = val[0] + bias;
            } else if (SLAI_EPI_IS(EPI_RESID)) {
                if (valid) P.out[orow] = e_resid + (val[0] + bias);
            } else if (SLAI_EPI_IS(EPI_XCHG)) {
                if (valid) {
                    float y = val[0] + bias;
                    if (P.xrank == 0) y += e_resid;
                    const uint2 pkt = make_uint2(__float_as_uint(y), xchg_seq(P, P.xo_idx1));
                    for (int rk = 0; rk < P.xr; rk++) P.xo_slot[rk][orow] = pkt;  // one 8-byte store each: value and tag together
                }
            } else if (SLAI_EPI_IS(EPI_SILU)) {
                if (valid) {
                    const float gt = val[0], up = val[NMAT - 1];
                    P.out[orow] = up * (gt / (1.0f + expf(-gt)));
                }
            } else if (SLAI_EPI_IS(EPI_GELU)) {
                if (valid) P.out[orow] = gelu_ref(val[0] + bias);
            } else if (SLAI_EPI_IS(EPI_QKV)) {
                float y = val[0] + bias;
                const int pos = P.pos1 > 0 ? P.pos1 - 1 : __ldcg(P.d_pos);
                // rows 2i, 2i+1 of a tile sit in neighbouring lanes of the same half-warp
                const float other = __shfl_xor_sync(__activemask(), y, 1);
                if (P.rope && sg.role < 2) {
                    const int hd = (row_in_seg & ~1) % P.head_size;
                    float sn, cs;
                    if (P.rope_cs) {
                        cs = e_cs;
                        sn = e_sn;
                    } else {
                        sincosf((float)pos * P.rope_theta[hd >> 1], &sn, &cs);
                    }
                    y = (r & 1) ? (sn * other + cs * y) : (cs * y - sn * other);
                }
                if (valid) {
                    if (sg.role == 0) {
                        P.out[orow] = y;
                    } else if (sg.role == 1 && P.k_out) {
                        P.k_out[row_in_seg] = y;
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
        SLAI_TRACE_POINT(12)
        if (wv + 1 < n_waves) {  // the partial buffer is reused by the next wave
            __syncthreads();
            for (int i = tid; i < WAVE * WARPS * NMAT * 16; i += THREADS) red[i] = 0.f;
            __syncthreads();
        }
    }
#undef SLAI_EPI_IS
}

}  // namespace gemvk

// gemv.cu: validate a launch description and turn it into kernel parameters (dig_region / nstage 0 = size them
// for this launch alone).
int gemv_fill_params(slai_ctx* ctx, const GemvLaunch& L, size_t dig_region, int nstage, gemvk::GemvParams& P, size_t* smem_out,
                     int* grid_out);
