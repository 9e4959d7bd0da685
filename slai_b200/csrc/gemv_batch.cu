// One pass over a quantised matrix for a batch of 2..8 input vectors (GemvQuant::launch with a matrix-shaped `v`,
// crates/slai/src/ops/gemv_quant.rs:206-312: the reference's shader loops over the columns inside one dispatch).
//
// The single-vector kernel (gemv.cu) spends the eight columns of the integer MMA on one vector (four digit planes x two
// sub-blocks); looping it over a batch streams the matrix once per vector.  Here the packed weights of a tile-step block
// are loaded and unpacked into MMA operands once and every vector of the batch adds its own MMAs
// (`compute_batch`, gemv_formats.cuh: per vector the same integer arithmetic as the single-vector code).
//
// Shape.  The digit planes of 8 vectors over the whole of K do not fit in shared memory, so K is cut into chunks of
// `ch` tile-steps (<= 8) and a unit of work is (chunk, group of 16 row tiles): the 16 warps of a block stage the chunk's
// slice of all vectors once (each vector with its own power-of-two scale for the chunk), then every warp walks its own
// tile's `ch` blocks, double-buffered with cp.async.  Partial sums per chunk go to a scratch array and a second small
// kernel adds them in chunk order (deterministic; no atomics).
#include <stdlib.h>

#include "common.cuh"
#include "gemv_formats.cuh"
#include "layout.cuh"

namespace {

using namespace gemvfmt;
using namespace frag;

constexpr int BWARPS = 16;
constexpr int BTHREADS = 32 * BWARPS;
constexpr int MAX_CH = 8;
constexpr int BSMEM_LIMIT = 227 * 1024;

struct BatchParams {
    const uint8_t* w[3];   // up to three matrices of the same format and K that share the input (q / k / v, gate / up): their
    int t0[3];             // 16-row tiles form one tile space, matrix i starts at tile t0[i]
    int nw;
    long long tile_bytes;
    int ntiles, nsteps, K;
    int ch, nch, ngroups;  // steps per chunk, chunks, groups of 16 tiles
    int n_batch;           // vectors that exist (the others of the instantiation's NV are zero)
    const float* v;        // [n_batch][K]
    float* part;           // [nch][NV][mp] partial sums
    int mp;                // ntiles * 16
    uint32_t plane;        // bytes between the digit planes of a staged vector (chunk elements + 32)
    uint32_t vstride;      // bytes between the staged vectors (digit planes, then the digit sums)
};

template <class F>
struct BatchGeom {
    static constexpr uint32_t STEP = F::STEP_BYTES;
    static constexpr uint32_t STRIDE = (STEP + 127) & ~127u;
};

__device__ __forceinline__ float bmax4(const float4& x) { return fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))); }

// One tile-step block, global -> this warp's stage: 16 bytes per lane and round.
template <class F>
__device__ __forceinline__ void stage_request(const uint8_t* src, uint32_t dst, int lane) {
    const size_t gsrc = __cvta_generic_to_global(src);
#pragma unroll 1
    for (uint32_t off = 16u * lane; off < BatchGeom<F>::STEP; off += 512u)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + off), "l"(gsrc + off) : "memory");
}
__device__ __forceinline__ void stage_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// NV vectors are staged; a tile-step block is taken against NC of them at a time (NV / NC passes over the block in shared
// memory: fewer accumulators live at once).
template <class F, int NV, int NC = NV>
__global__ void __launch_bounds__(BTHREADS, 1) gemv_batch_kernel(const __grid_constant__ BatchParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    Smem S;
    S.zero = sbase;
    S.dig = sbase + ZERO_BYTES;
    S.plane = P.plane;
    S.sv = S.dig + 4 * P.plane;
    const uint32_t misc_off = ZERO_BYTES + NV * P.vstride;
    float* sinv = reinterpret_cast<float*>(smem + misc_off);                 // 1 / scale of every staged vector
    unsigned int* smax = reinterpret_cast<unsigned int*>(smem + misc_off + 32);  // max |x| of the chunk per vector, as float bits
    const uint32_t ring_off = (misc_off + 64 + 127) & ~127u;
    const uint32_t wb = sbase + ring_off + (uint32_t)warp * 2u * BatchGeom<F>::STRIDE;

    LaneCtx L;
    lane_init<F>(L, lane, S);
    const uint32_t bvs = L.bmul ? P.vstride : 0u;  // lanes that read the zero page read it for every vector

    if (tid < ZERO_BYTES / 4) reinterpret_cast<uint32_t*>(smem)[tid] = 0u;
    if (tid < NV) smax[tid] = 0u;

    const int ce = P.ch * F::STEP;  // elements of K per chunk
    const int per = ce >> 5;        // sub-blocks of 32 elements per vector and chunk (<= 64)
    const int sv_v = tid / per, sv_j = tid - sv_v * per;  // the (vector, sub-block) this thread stages
    const bool stager = sv_v < NV;

    const int units = P.ngroups * P.nch;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        const int c = unit / P.ngroups, grp = unit - c * P.ngroups;
        const int s0 = c * P.ch;
        const int nst = min(P.ch, P.nsteps - s0);
        const int tile = grp * BWARPS + warp;
        const bool active = tile < P.ntiles;
        const uint8_t* wbase = P.w[0];
        int wt0 = 0;
        if (P.nw > 1 && tile >= P.t0[1]) { wbase = P.w[1]; wt0 = P.t0[1]; }
        if (P.nw > 2 && tile >= P.t0[2]) { wbase = P.w[2]; wt0 = P.t0[2]; }
        const uint8_t* src = wbase + (size_t)(active ? tile - wt0 : 0) * P.tile_bytes + (size_t)s0 * BatchGeom<F>::STEP;
        // the first two blocks of this warp's tile are on their way while the vectors are staged
        if (active) stage_request<F>(src, wb, lane);
        stage_commit();
        if (active && nst > 1) stage_request<F>(src + BatchGeom<F>::STEP, wb + BatchGeom<F>::STRIDE, lane);
        stage_commit();

        // ---- stage the chunk's slice of every vector: thread (vector, sub-block of 32 elements) ----
        float4 x[8];
        {
            const int k0 = s0 * F::STEP + 32 * sv_j;
            const bool have = stager && sv_v < P.n_batch && k0 < P.K;
            const float4* p = reinterpret_cast<const float4*>(P.v + (size_t)(have ? sv_v : 0) * P.K + (have ? k0 : 0));
            float mx = 0.f;
#pragma unroll
            for (int e = 0; e < 8; e++) {
                x[e] = have ? __ldcg(p + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                mx = fmaxf(mx, bmax4(x[e]));
            }
            __syncthreads();  // every warp has finished the previous unit (digits, sums and `smax` are free)
            if (stager && mx > 0.f) atomicMax(&smax[sv_v], __float_as_uint(mx));
        }
        __syncthreads();
        if (stager) {
            const float mx = __uint_as_float(smax[sv_v]);
            float scale = 1.f;
            if (mx > 0.f && mx < 3.0e38f) {
                int e = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 126;  // mx = f * 2^e with f in [0.5, 1) (normal numbers)
                if ((__float_as_uint(mx) >> 23) == 0u) e = -126;
                e = e < -90 ? -90 : e;
                scale = __uint_as_float((uint32_t)(127 + 26 - e) << 23);  // 2^(26 - e), exact
            }
            if (sv_j == 0) sinv[sv_v] = 1.0f / scale;
            unsigned char* dig = smem + ZERO_BYTES + (size_t)sv_v * P.vstride;
            unsigned char* svb = dig + 4 * (size_t)P.plane;
            uint32_t pw[8][4];
#pragma unroll
            for (int e = 0; e < 8; e++)
                digit_planes(digits_word(__float2int_rn(x[e].x * scale)), digits_word(__float2int_rn(x[e].y * scale)),
                             digits_word(__float2int_rn(x[e].z * scale)), digits_word(__float2int_rn(x[e].w * scale)), pw[e]);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                uint4* d = reinterpret_cast<uint4*>(dig + (size_t)q * P.plane + 32 * sv_j);
                d[0] = make_uint4(pw[0][q], pw[1][q], pw[2][q], pw[3][q]);
                d[1] = make_uint4(pw[4][q], pw[5][q], pw[6][q], pw[7][q]);
            }
            if (F::SV_GRAN == 32) {
                // Q4_K / Q5_K: sum of the sub-block's digits per plane as two base-128 digits in the byte table of its step
                unsigned char* tab = svb + (sv_j >> 3) * 128;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    int sd = 0;
#pragma unroll
                    for (int e = 0; e < 8; e++) sd = __dp4a((int)pw[e][q], 0x01010101, sd);
                    const int hi = (sd + 64) >> 7, lo = sd - (hi << 7);
                    tab[(2 * q) * 16 + (sv_j & 7)] = (unsigned char)hi;
                    tab[(2 * q + 1) * 16 + (sv_j & 7)] = (unsigned char)lo;
                }
                *reinterpret_cast<uint2*>(tab + (sv_j & 7) * 16 + 8) = make_uint2(0u, 0u);
            } else if (F::SV_GRAN == 16) {
                // Q6_K: 4 x s32 per sub-block of 16 elements
                int4* sv = reinterpret_cast<int4*>(svb);
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    int sd[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        sd[q] = 0;
#pragma unroll
                        for (int e = 0; e < 4; e++) sd[q] = __dp4a((int)pw[4 * half + e][q], 0x01010101, sd[q]);
                    }
                    sv[2 * sv_j + half] = make_int4(sd[0], sd[1], sd[2], sd[3]);
                }
            }
        }
        __syncthreads();
        if (tid < NV) smax[tid] = 0u;  // read by everyone before the barrier above; next written after the next unit's first barrier

        // ---- this warp's tile: `nst` blocks against all vectors ----
        float accA[NV], accB[NV];
#pragma unroll
        for (int v = 0; v < NV; v++) accA[v] = accB[v] = 0.f;
        if (active) {
#pragma unroll 1
            for (int s = 0; s < nst; s++) {
                asm volatile("cp.async.wait_group 1;" ::: "memory");  // all but the newest request have landed: block s is here
                __syncwarp();
                const uint32_t blk = wb + (uint32_t)(s & 1) * BatchGeom<F>::STRIDE;
                if (NC == NV) {
                    F::template compute_batch<NV>(blk, s, L, S, bvs, P.vstride, accA, accB);
                } else {
#pragma unroll
                    for (int pass = 0; pass < NV / NC; pass++) {
                        LaneCtx L2 = L;
                        L2.bbase += (uint32_t)(pass * NC) * bvs;
                        Smem S2 = S;
                        S2.sv += (uint32_t)(pass * NC) * P.vstride;
                        F::template compute_batch<NC>(blk, s, L2, S2, bvs, P.vstride, reinterpret_cast<float(&)[NC]>(accA[pass * NC]),
                                                      reinterpret_cast<float(&)[NC]>(accB[pass * NC]));
                    }
                }
                __syncwarp();
                if (s + 2 < nst) stage_request<F>(src + (size_t)(s + 2) * BatchGeom<F>::STEP, blk, lane);
                stage_commit();
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
        for (int v = 0; v < NV; v++) {
            accA[v] += __shfl_xor_sync(0xffffffffu, accA[v], 1);
            accA[v] += __shfl_xor_sync(0xffffffffu, accA[v], 2);
            accB[v] += __shfl_xor_sync(0xffffffffu, accB[v], 1);
            accB[v] += __shfl_xor_sync(0xffffffffu, accB[v], 2);
        }
        if (active) {
#pragma unroll
            for (int v = 0; v < NV; v++)
                if ((v & 3) == L.t) {  // the four lanes of a row hold the same sums: lane t stores vectors t and t + 4
                    const float inv = sinv[v];
                    float* dst = P.part + ((size_t)c * NV + v) * P.mp + (size_t)tile * 16;
                    dst[L.g] = accA[v] * inv;
                    dst[L.g + 8] = accB[v] * inv;
                }
        }
    }
}

// out[v][m] = sum over the chunks, in order, of the partial sums.
// epi: BATCH_STORE, BATCH_ADD (out += sum: the residual streams of the batch), BATCH_SILU (out = sum * silu(gate), gate laid
// out like out: ops/silu.rs:50-58 with the sum as h2 and gate as h1), BATCH_PAIR_SILU (two matrices of M rows each in one
// launch, gate then up: out = up sum * silu(gate sum)).
__global__ void gemv_batch_reduce_kernel(float* out, long long ldo, const float* part, int nch, int nv, int mp, int M, int n_batch, int epi,
                                         const float* gate) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_batch * M) return;
    const int v = (int)(idx / M), m = (int)(idx - (long long)v * M);
    float s = 0.f;
    for (int c = 0; c < nch; c++) s += part[((size_t)c * nv + v) * mp + m];
    const long long o = (long long)v * ldo + m;
    if (epi == BATCH_ADD) {
        s = out[o] + s;
    } else if (epi == BATCH_SILU) {
        const float g = gate[o];
        s = s * (g / (1.0f + expf(-g)));
    } else if (epi == BATCH_PAIR_SILU) {
        float u = 0.f;
        for (int c = 0; c < nch; c++) u += part[((size_t)c * nv + v) * mp + M + m];
        s = u * (s / (1.0f + expf(-s)));
    }
    out[o] = s;
}

template <class F>
size_t batch_smem(int nv, int ch, uint32_t* plane_out, uint32_t* vstride_out) {
    const uint32_t ce = (uint32_t)ch * F::STEP;
    const uint32_t plane = ce + 32;
    const uint32_t svbytes = F::SV_GRAN == 32 ? 128u * ch : F::SV_GRAN == 16 ? ce : 0u;
    const uint32_t vstride = (4 * plane + svbytes + 15) & ~15u;
    *plane_out = plane;
    *vstride_out = vstride;
    const uint32_t ring_off = (ZERO_BYTES + nv * vstride + 64 + 127) & ~127u;
    return (size_t)ring_off + (size_t)BWARPS * 2 * BatchGeom<F>::STRIDE;
}

template <class F, int NV, int NC = NV>
int launch_batch_inst(slai_ctx* ctx, BatchParams& P, float* d_out, long long ldo, int M, int epi, const float* gate) {
    // Steps per chunk: the fewest rounds of (staging + ch steps) over the SMs; staging a chunk costs about three steps.
    const int G = ctx->sm_count > 0 ? ctx->sm_count : 148;
    int best_ch = 1;
    long long best_cost = -1;
    for (int ch = 1; ch <= MAX_CH; ch++) {
        const long long nch = (P.nsteps + ch - 1) / ch;
        const long long rounds = (nch * P.ngroups + G - 1) / G;
        const long long cost = rounds * (3 + ch);
        if (best_cost < 0 || cost <= best_cost) {
            best_cost = cost;
            best_ch = ch;
        }
    }
    P.ch = best_ch;
    P.nch = (P.nsteps + P.ch - 1) / P.ch;
    const size_t smem = batch_smem<F>(NV, P.ch, &P.plane, &P.vstride);
    SLAI_REQUIRE(ctx, smem <= (size_t)BSMEM_LIMIT, SLAI_ERR_SHAPE, "gemv: the batched kernel needs %zu bytes of shared memory", smem);
    const size_t part_bytes = (size_t)P.nch * NV * P.mp * sizeof(float);
    int rc = ensure_scratch(ctx, part_bytes);
    if (rc) return rc;
    P.part = reinterpret_cast<float*>(ctx->d_scratch);
    auto kern = gemv_batch_kernel<F, NV, NC>;
    static PerDeviceOnce attr;  // per instantiation
    if (attr.need(ctx->device)) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BSMEM_LIMIT));
        attr.set(ctx->device);
    }
    const long long units = (long long)P.ngroups * P.nch;
    const int grid = (int)(units < G ? units : G);
    kern<<<grid, BTHREADS, smem, ctx->stream>>>(P);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    const long long total = (long long)P.n_batch * M;
    gemv_batch_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(d_out, ldo, P.part, P.nch, NV, P.mp, M, P.n_batch, epi, gate);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}

template <class F>
int launch_batch_fmt(slai_ctx* ctx, BatchParams& P, float* d_out, long long ldo, int M, int epi, const float* gate) {
    if (P.n_batch <= 2) return launch_batch_inst<F, 2>(ctx, P, d_out, ldo, M, epi, gate);
    if (P.n_batch <= 4) return launch_batch_inst<F, 4>(ctx, P, d_out, ldo, M, epi, gate);
    // Eight vectors: a block is taken against four of them at a time (two passes over it in shared memory) -- with all
    // eight at once the accumulators leave the compiler no registers to overlap loads and MMAs (measured 7 % slower on
    // the 11008-wide shapes).  SLAI_BATCH_PASSES=1 selects the one-pass kernel.
    static const int passes = [] { const char* e = getenv("SLAI_BATCH_PASSES"); return e ? atoi(e) : 2; }();
    if (passes != 1) return launch_batch_inst<F, 8, 4>(ctx, P, d_out, ldo, M, epi, gate);
    return launch_batch_inst<F, 8>(ctx, P, d_out, ldo, M, epi, gate);
}

}  // namespace

bool gemv_batch_supported(const slai_qmatrix* w) {
    return w->fmt == SLAI_FMT_Q8_0 || w->fmt == SLAI_FMT_Q4_K || w->fmt == SLAI_FMT_Q5_K || w->fmt == SLAI_FMT_Q6_K;
}

// out[b * ldo + m] = sum_k W[m][k] v[b][k] for b < n_batch (2..8), one pass over W (ldo 0: the rows of `out` are M apart);
// `epi` folds a residual add or the SiLU gate into the store.  W is the concatenation by rows of `nw` (1..3) matrices of the
// same format and width (all but the last with a multiple of 16 rows); with BATCH_PAIR_SILU the two matrices are gate and up
// of equal height M and out[b * ldo + m], m < M, receives up * silu(gate).
int gemv_batch_launch_multi(slai_ctx* ctx, float* d_out, const slai_qmatrix* const* ws, int nw, const float* d_v, int n_batch, long long ldo,
                            int epi, const float* d_gate) {
    SLAI_REQUIRE(ctx, nw >= 1 && nw <= 3 && ws && ws[0], SLAI_ERR_INVALID_ARG, "gemv: %d matrices in one batched launch", nw);
    const slai_qmatrix* w = ws[0];
    SLAI_REQUIRE(ctx, gemv_batch_supported(w), SLAI_ERR_UNSUPPORTED_FORMAT, "gemv: format %d has no batched kernel", w->fmt);
    SLAI_REQUIRE(ctx, n_batch >= 2 && n_batch <= 8, SLAI_ERR_INVALID_ARG, "gemv: batch of %d", n_batch);
    SLAI_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(d_v) & 15) == 0, SLAI_ERR_INVALID_ARG, "gemv: the input vectors must be 16-byte aligned");
    BatchParams P = {};
    int rows_total = 0, tiles = 0;
    for (int i = 0; i < nw; i++) {
        SLAI_REQUIRE(ctx, ws[i] && ws[i]->fmt == w->fmt && ws[i]->ncols == w->ncols && ws[i]->tile_bytes == w->tile_bytes, SLAI_ERR_SHAPE,
                     "gemv: matrices of one batched launch must share format and width");
        SLAI_REQUIRE(ctx, i == nw - 1 || ws[i]->nrows % 16 == 0, SLAI_ERR_SHAPE, "gemv: %lld rows before another matrix of the launch",
                     (long long)ws[i]->nrows);
        SLAI_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(ws[i]->data) & 15) == 0 && ws[i]->tile_bytes % 16 == 0, SLAI_ERR_INVALID_ARG,
                     "gemv: matrix data must be 16-byte aligned");
        P.w[i] = ws[i]->data;
        P.t0[i] = tiles;
        tiles += (int)layout::num_tiles(ws[i]->nrows);
        rows_total += (int)ws[i]->nrows;
    }
    P.nw = nw;
    P.tile_bytes = w->tile_bytes;
    P.ntiles = tiles;
    P.nsteps = (int)layout::num_steps(w->fmt, w->ncols);
    P.K = (int)w->ncols;
    P.ngroups = (P.ntiles + BWARPS - 1) / BWARPS;
    P.n_batch = n_batch;
    P.v = d_v;
    P.mp = P.ntiles * 16;
    int M = rows_total;
    if (epi == BATCH_PAIR_SILU) {
        SLAI_REQUIRE(ctx, nw == 2 && ws[0]->nrows == ws[1]->nrows, SLAI_ERR_SHAPE, "gemv: the gate / up epilogue takes two matrices of equal height");
        M = (int)ws[0]->nrows;
    }
    if (ldo <= 0) ldo = M;
    SLAI_REQUIRE(ctx, ldo >= M, SLAI_ERR_SHAPE, "gemv: output rows %lld apart hold fewer than %d values", ldo, M);
    SLAI_REQUIRE(ctx, epi == BATCH_STORE || epi == BATCH_ADD || epi == BATCH_PAIR_SILU || (epi == BATCH_SILU && d_gate), SLAI_ERR_INVALID_ARG,
                 "gemv: batch epilogue %d", epi);
    switch (w->fmt) {
        case SLAI_FMT_Q8_0: return launch_batch_fmt<Q80>(ctx, P, d_out, ldo, M, epi, d_gate);
        case SLAI_FMT_Q4_K: return launch_batch_fmt<Q4K>(ctx, P, d_out, ldo, M, epi, d_gate);
        case SLAI_FMT_Q5_K: return launch_batch_fmt<Q5K>(ctx, P, d_out, ldo, M, epi, d_gate);
        case SLAI_FMT_Q6_K: return launch_batch_fmt<Q6K>(ctx, P, d_out, ldo, M, epi, d_gate);
    }
    return SLAI_ERR_UNSUPPORTED_FORMAT;
}

int gemv_batch_launch(slai_ctx* ctx, float* d_out, const slai_qmatrix* w, const float* d_v, int n_batch, long long ldo, int epi,
                      const float* d_gate) {
    return gemv_batch_launch_multi(ctx, d_out, &w, 1, d_v, n_batch, ldo, epi, d_gate);
}
