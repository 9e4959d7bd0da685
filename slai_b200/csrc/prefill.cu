// Prompt processing as dense contractions on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// The reference feeds a prompt one token at a time through its decode step (crates/slai-chat/src/chat_llama2.rs:109-115
// loops forward_logits over the prompt; the operator sequence is Llama2::launch, crates/slai/src/models/llama2/
// transformer.rs:316-381).  For a prompt of T tokens that streams every weight T times.  Here the T activation rows go
// through each matrix together: Y[T x M] = X[T x K] W^T, the only place on this path where the work is a GEMM.
//
// Numerics.  Parity with the sequential path is the contract (logits and KV cache within 1e-3 relative L2, same greedy
// continuation), and a single fp16 rounding of both operands per product (4e-4 per GEMM, compounding over 4 GEMMs x
// layers) would spend that budget.  Both operands are therefore carried as fp16 pairs, v = hi + lo with
// hi = fp16(v), lo = fp16(v - hi) (22 significant bits), and every 16-deep product is issued three times
// (hi*hi, hi*lo, lo*hi) into the same f32 accumulator: about 2^-21 per product, the rest of the error is the f32
// accumulation order.  The tensor cores have the headroom: the kernel is bound by dequantisation, not by MMA issue.
//
// One CTA computes a 128 (weight rows) x NT (tokens, <= 256) tile of Y^T over the whole K:
//   * warps 2-9 (256 threads, two per weight row, one 32-element half of the slice each): read the row's packed quants
//     of the next 64-element K slice from the tile-major matrix (the decode layout, layout.cuh) one stage ahead of their
//     use, dequantise with the reference's rounding sequence, split into hi / lo and store them into the A operand
//     tiles in the canonical K-major 128-byte-swizzled layout;
//   * warp 0, one lane: TMA (cp.async.bulk.tensor.2d, no multicast: the tile is this CTA's own) brings the matching
//     64-element slice of the activations' hi and lo planes [T_pad x K] into the B operand tiles, same swizzle;
//   * warp 1, one lane: issues tcgen05.mma (kind::f16, M = 128, N = NT, K = 16) four slices x three products per stage
//     and commits the stage's completion to an mbarrier, which frees the stage for the producers;
//   * epilogue (warps 2-9 again): tcgen05.ld brings each thread one accumulator row (32 TMEM lanes per warp, the
//     quadrant given by warp index mod 4; the two warps of a quadrant take alternate groups of 16 tokens), adds bias /
//     residual and stores Y[t][row] with coalesced 128-byte rows.
// Two stages of A and B (192 KB of shared memory at NT = 256), 1 CTA per SM, TMEM columns = NT rounded to a power of two.
// Every mbarrier wait is bounded: on expiry the error flag is raised and the role leaves its loop; all roles then meet
// at the final barrier and the tensor memory is released.
#include <cuda.h>

#include "common.cuh"
#include "dequant.cuh"

namespace {

constexpr int PF_DQ_THREADS = 256;  // dequantising threads: two per weight row (one 32-element sub-block each)
constexpr int PF_THREADS = 64 + PF_DQ_THREADS;
constexpr int PF_BM = 128;          // weight rows per CTA
constexpr int PF_BK = 64;           // K elements per stage (one 128-byte swizzle row of fp16)
constexpr int PF_STAGES = 2;
constexpr int PF_A_BYTES = PF_BM * PF_BK * 2;  // one A plane of a stage

struct PrefillGemmParams {
    const uint8_t* w;        // tile-major quantised matrix
    long long tile_bytes;    // bytes of one 16-row tile (all K steps)
    int fmt, M, K;           // matrix rows and columns
    int T, NT;               // valid tokens, tokens per CTA tile (multiple of 16, <= 256)
    float* out;              // [T][ldo]; row m goes to out[t * ldo + out_off + m]
    int ldo, out_off;
    const float* resid;      // optional [T][ldr]: out = resid + y (may alias out)
    int ldr;
    const float* bias;       // optional [M]
    unsigned int* err_flag;
    unsigned int wait_limit;
};

// ---- PTX wrappers ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t a, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(a), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Bounded wait: false (and the error flag raised) if the phase does not complete.
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity, const PrefillGemmParams& P) {
    for (unsigned int i = 0; i < P.wait_limit; i++) {
        if (mbar_try(a, parity)) return true;
        if (i > 64) __nanosleep(40);
    }
    atomicExch(P.err_flag, 5u);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(mbar), "r"(x), "r"(y)
                 : "memory");
}
// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled operand tile (rows of 64 fp16 = 128 bytes, 8-row
// groups 1024 bytes apart): start address / 16 in bits 0-13, leading offset (unused with this swizzle) 1 in bits 16-29,
// stride between 8-row groups / 16 in bits 32-45, descriptor version 1 in bits 46-47, swizzle mode 2 (128 B) in bits 61-63.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: f32 accumulator (bits 4-5 = 1), A and B fp16 (0), both K-major (bits 15, 16 = 0),
// N / 8 in bits 17-22, M / 16 in bits 24-28.
__device__ __forceinline__ uint32_t umma_idesc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(PF_BM >> 4) << 24); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// 64 dequantised values of one row into its 128-byte rows of the hi and lo A planes.  Chunk c (8 values, 16 bytes) of
// row r lives at chunk position c ^ (r & 7) of the row (the 128-byte swizzle the tensor core expects).
__device__ __forceinline__ void store_split8(unsigned char* a_hi, unsigned char* a_lo, int r, int c, const float (&v)[8]) {
    __half2 h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half h0 = __float2half_rn(v[2 * i]), h1 = __float2half_rn(v[2 * i + 1]);
        h[i] = __halves2half2(h0, h1);
        l[i] = __halves2half2(__float2half_rn(v[2 * i] - __half2float(h0)), __float2half_rn(v[2 * i + 1] - __half2float(h1)));
    }
    const int off = r * 128 + ((c ^ (r & 7)) << 4);
    *reinterpret_cast<uint4*>(a_hi + off) = *reinterpret_cast<const uint4*>(h);
    *reinterpret_cast<uint4*>(a_lo + off) = *reinterpret_cast<const uint4*>(l);
}

// Half `part` (32 elements = one sub-block of Q4_K / Q5_K) of the slice [k0, k0 + 64) of row `row`.  For Q4_K / Q5_K the
// and one 32-element block of Q8_0 the packed bytes are fetched into registers (`slice_fetch`) a stage before they are
// turned into operand rows (`slice_emit`), so that the loads' latency runs behind the previous stage's arithmetic; Q6_K
// goes element by element.
struct SliceRegs {
    uint4 q[2], hq[2];     // the 32 nibble bytes of the 64-element group, the row's 32 high-bit bytes (Q5_K)
    uint32_t dd, sc, mb;   // f16 d | f16 dmin, scale and minimum of this thread's sub-block
};
__device__ __forceinline__ void slice_fetch(const PrefillGemmParams& P, long long row, int k0, int part, SliceRegs& R) {
    if (P.fmt == SLAI_FMT_Q8_0) {  // a step is four 32-element blocks; this thread's block is 32 consecutive bytes of the lane-ordered region
        const int r16 = (int)(row & 15), e = (k0 & 127) + 32 * part, b8 = e >> 5;
        const uint8_t* b = P.w + (row >> 4) * P.tile_bytes + (long long)(k0 >> 7) * 2176;
        R.dd = __ldg(reinterpret_cast<const unsigned short*>(b + 8 * r16 + 2 * b8));
        const uint4* q = reinterpret_cast<const uint4*>(b + layout::qbyte_off(128, r16, 32 * b8));
        R.q[0] = __ldg(q);
        R.q[1] = __ldg(q + 1);
        return;
    }
    const bool five = P.fmt == SLAI_FMT_Q5_K;
    const int r16 = (int)(row & 15), G = (k0 >> 6) & 3;
    const uint8_t* b = P.w + (row >> 4) * P.tile_bytes + (long long)(k0 >> 8) * layout::step_bytes(P.fmt);
    const uint8_t* h = b + layout::K45_HDR_ROW * r16;
    const int j = 2 * G + part;
    R.dd = __ldg(reinterpret_cast<const uint32_t*>(h));
    R.sc = __ldg(h + layout::k45_sc_off(j));
    R.mb = __ldg(h + 12 + j);
    const int q0 = five ? layout::K45_HDR + 512 : layout::K45_HDR;
    R.q[0] = __ldg(reinterpret_cast<const uint4*>(b + layout::qbyte_off(q0, r16, 32 * G)));
    R.q[1] = __ldg(reinterpret_cast<const uint4*>(b + layout::qbyte_off(q0, r16, 32 * G + 16)));
    if (five) {
        R.hq[0] = __ldg(reinterpret_cast<const uint4*>(b + layout::K45_HDR + 32 * r16));
        R.hq[1] = __ldg(reinterpret_cast<const uint4*>(b + layout::K45_HDR + 32 * r16 + 16));
    }
}
__device__ __forceinline__ void slice_emit(const PrefillGemmParams& P, const SliceRegs& R, int r, int k0, int part, unsigned char* a_hi,
                                           unsigned char* a_lo) {
    if (P.fmt == SLAI_FMT_Q8_0) {  // q * scale (quantization.rs:38-41)
        const float d = dev_h2f(R.dd);
        const uint32_t qw8[8] = {R.q[0].x, R.q[0].y, R.q[0].z, R.q[0].w, R.q[1].x, R.q[1].y, R.q[1].z, R.q[1].w};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int l = 8 * c + i;
                v[i] = __fmul_rn((float)(int)(signed char)((qw8[l >> 2] >> (8 * (l & 3))) & 0xFFu), d);
            }
            store_split8(a_hi, a_lo, r, 4 * part + c, v);
        }
        return;
    }
    const bool five = P.fmt == SLAI_FMT_Q5_K;
    const int G = (k0 >> 6) & 3;
    const float d1 = __fmul_rn(dev_h2f(R.dd & 0xFFFFu), (float)R.sc), m1 = __fmul_rn(dev_h2f(R.dd >> 16), (float)R.mb);
    const uint32_t qw[8] = {R.q[0].x, R.q[0].y, R.q[0].z, R.q[0].w, R.q[1].x, R.q[1].y, R.q[1].z, R.q[1].w};
    const uint32_t hw[8] = {R.hq[0].x, R.hq[0].y, R.hq[0].z, R.hq[0].w, R.hq[1].x, R.hq[1].y, R.hq[1].z, R.hq[1].w};
#pragma unroll
    for (int c = 0; c < 4; c++) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int l = 8 * c + i;  // element of the sub-block = byte l of the group
            int q = (int)((qw[l >> 2] >> (8 * (l & 3) + 4 * part)) & 0xFu);
            if (five) q += (int)((hw[l >> 2] >> (8 * (l & 3) + 2 * G + part)) & 1u) << 4;
            v[i] = __fsub_rn(__fmul_rn(d1, (float)q), m1);
        }
        store_split8(a_hi, a_lo, r, 4 * part + c, v);
    }
}
__device__ __forceinline__ void slice_generic(const PrefillGemmParams& P, long long row, int r, int k0, int part, unsigned char* a_hi,
                                              unsigned char* a_lo) {
#pragma unroll 1
    for (int c = 4 * part; c < 4 * part + 4; c++) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = row < P.M ? dequant_elem(P.fmt, P.w, P.K, row, k0 + 8 * c + i) : 0.f;  // rows beyond the matrix: zeros
        store_split8(a_hi, a_lo, r, c, v);
    }
}

__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_gemm_kernel(const __grid_constant__ PrefillGemmParams P, const __grid_constant__ CUtensorMap map_hi,
                    const __grid_constant__ CUtensorMap map_lo) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    const int NT = P.NT;
    const int b_bytes = NT * PF_BK * 2;  // one B plane of a stage
    unsigned char* a_hi = smem;                              // [stage][128 x 128 B]
    unsigned char* a_lo = a_hi + PF_STAGES * PF_A_BYTES;
    unsigned char* b_hi = a_lo + PF_STAGES * PF_A_BYTES;     // [stage][NT x 128 B]
    unsigned char* b_lo = b_hi + PF_STAGES * b_bytes;
    __shared__ __align__(8) unsigned long long bars[3 * PF_STAGES + 1];
    __shared__ uint32_t tmem_slot;
    const uint32_t full_a = smem_u32(&bars[0]), full_b = smem_u32(&bars[PF_STAGES]), empty = smem_u32(&bars[2 * PF_STAGES]),
                   accum = smem_u32(&bars[3 * PF_STAGES]);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * PF_BM, n0 = blockIdx.y * NT;
    const int nk = P.K / PF_BK;
    int ncols = 32;
    while (ncols < NT) ncols <<= 1;

    if (tid == 0) {
        for (int s = 0; s < PF_STAGES; s++) {
            mbar_init(full_a + 8 * s, PF_DQ_THREADS);
            mbar_init(full_b + 8 * s, 1);
            mbar_init(empty + 8 * s, 1);
        }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;

    if (warp == 0) {
        // ---- activations: one lane drives the TMA ----
        if (lane == 0) {
            for (int s = 0; s < nk; s++) {
                const int st = s % PF_STAGES;
                if (s >= PF_STAGES && !mbar_wait(empty + 8 * st, ((s / PF_STAGES) - 1) & 1, P)) break;
                mbar_expect_tx(full_b + 8 * st, 2 * b_bytes);
                tma_load_2d(smem_u32(b_hi + st * b_bytes), &map_hi, s * PF_BK, n0, full_b + 8 * st);
                tma_load_2d(smem_u32(b_lo + st * b_bytes), &map_lo, s * PF_BK, n0, full_b + 8 * st);
            }
        }
    } else if (warp == 1) {
        // ---- tensor cores: one lane issues, the stage is handed back when its products have been read ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(NT);
            bool ok = true;
            for (int s = 0; s < nk && ok; s++) {
                const int st = s % PF_STAGES;
                const uint32_t par = (s / PF_STAGES) & 1;
                ok = mbar_wait(full_a + 8 * st, par, P) && mbar_wait(full_b + 8 * st, par, P);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t ah = smem_u32(a_hi + st * PF_A_BYTES), al = smem_u32(a_lo + st * PF_A_BYTES);
                const uint32_t bh = smem_u32(b_hi + st * b_bytes), bl = smem_u32(b_lo + st * b_bytes);
#pragma unroll
                for (int kk = 0; kk < PF_BK / 16; kk++) {  // 16 elements = 32 bytes further along the swizzled row
                    const uint64_t dah = umma_desc(ah + 32 * kk), dal = umma_desc(al + 32 * kk);
                    const uint64_t dbh = umma_desc(bh + 32 * kk), dbl = umma_desc(bl + 32 * kk);
                    umma_f16(tmem_d, dah, dbh, idesc, (s > 0 || kk > 0) ? 1u : 0u);
                    umma_f16(tmem_d, dah, dbl, idesc, 1u);
                    umma_f16(tmem_d, dal, dbh, idesc, 1u);
                }
                umma_commit(empty + 8 * st);
            }
            umma_commit(accum);  // arrives when everything issued above has completed (also after a bail-out)
        }
    } else {
        // ---- weights: two threads per row, dequantised into the A planes ----
        const int r = (tid - 64) & (PF_BM - 1), part = (tid - 64) >> 7;
        const long long row = (long long)m0 + r;
        const bool fast = (P.fmt == SLAI_FMT_Q4_K || P.fmt == SLAI_FMT_Q5_K || P.fmt == SLAI_FMT_Q8_0) && row < P.M;
        SliceRegs cur = {}, nxt = {};
        if (fast) slice_fetch(P, row, 0, part, cur);
        bool ok = true;
        for (int s = 0; s < nk && ok; s++) {
            const int st = s % PF_STAGES;
            if (fast && s + 1 < nk) slice_fetch(P, row, (s + 1) * PF_BK, part, nxt);  // in flight during the wait and the arithmetic
            if (s >= PF_STAGES) ok = mbar_wait(empty + 8 * st, ((s / PF_STAGES) - 1) & 1, P);
            if (!ok) break;
            if (fast) slice_emit(P, cur, r, s * PF_BK, part, a_hi + st * PF_A_BYTES, a_lo + st * PF_A_BYTES);
            else slice_generic(P, row, r, s * PF_BK, part, a_hi + st * PF_A_BYTES, a_lo + st * PF_A_BYTES);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core's reads
            mbar_arrive(full_a + 8 * st);
            cur = nxt;
        }
        // ---- epilogue: this thread's accumulator row, 16 tokens at a time ----
        if (mbar_wait(accum, 0, P)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int quad = warp & 3;              // a warp reads the 32 TMEM lanes of its quadrant
            const int colpart = (warp - 2) >> 2;    // the two warps of a quadrant take alternate groups of 16 tokens
            const int orow = m0 + 32 * quad + lane;
            const float bias = (P.bias && orow < P.M) ? P.bias[orow] : 0.f;
            for (int c0 = 16 * colpart; c0 < NT; c0 += 32) {
                uint32_t v[16];
                tmem_ld16(tmem_d + ((uint32_t)(32 * quad) << 16) + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (orow < P.M) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int t = n0 + c0 + j;
                        if (t < P.T) {
                            float y = __uint_as_float(v[j]) + bias;
                            if (P.resid) y = P.resid[(size_t)t * P.ldr + orow] + y;
                            P.out[(size_t)t * P.ldo + P.out_off + orow] = y;
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(ncols) : "memory");
}

// ---- causal attention of a block of prompt tokens ---------------------------------------------------------------------
// The decode step's attention serves one query token and streams that token's whole key / value history; run once per
// prompt token it reads the caches T / 2 times over.  Here one CTA takes 16 consecutive query tokens of one head and walks
// the positions they may attend to in tiles of 32: a tile of keys and values is brought into shared memory once (as f32)
// and serves all 16 queries.  Warp w owns queries 4w .. 4w + 3; for the scores lane = position of the tile (a 128-bit read
// of its own key row per four dimensions, the queries broadcast), then a streaming softmax per query (running maximum
// and sum, ops/batched_multiquery_attention.rs:102-156 computes the same softmax over all positions at once), then for the
// weighted sum of values lane = four output dimensions.  Plain f32 arithmetic, like the decode step's kernel.
constexpr int PA_QT = 16, PA_KT = 32, PA_THREADS = 128, PA_MAXC = 2;  // head_size <= 128 * PA_MAXC

template <typename T>
__device__ __forceinline__ void pa_load_rows(const T* __restrict__ g, long long row_stride, int rows, int hs, float* s, int s_stride, int tid) {
    constexpr int VEC = 16 / (int)sizeof(T);  // elements per 16-byte piece
    const int ppr = hs / VEC;
    for (int idx = tid; idx < PA_KT * ppr; idx += PA_THREADS) {
        const int r = idx / ppr, c = idx - r * ppr;
        float v[VEC];
        if (r < rows) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(g + (long long)r * row_stride) + c);
            if (sizeof(T) == 2) {
                const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                for (int i = 0; i < VEC / 2; i++) {
                    const float2 f = __half22float2(h2[i]);
                    v[2 * i] = f.x;
                    v[2 * i + 1] = f.y;
                }
            } else {
                const float* f = reinterpret_cast<const float*>(&raw);
#pragma unroll
                for (int i = 0; i < VEC; i++) v[i] = f[i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < VEC; i++) v[i] = 0.f;
        }
        float* dst = s + (size_t)r * s_stride + c * VEC;
#pragma unroll
        for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
}

template <typename T>
__global__ void __launch_bounds__(PA_THREADS)
prefill_attn_kernel(const float* __restrict__ q, int q_ld, const T* __restrict__ kc, const T* __restrict__ vc, long long head_stride, int hs, int kv_mul,
                    int pos0, int n_tokens, float* __restrict__ out, int out_ld) {
    extern __shared__ __align__(16) float pa_sm[];
    const int ks = hs + 4;              // key rows 4 floats apart modulo 32 banks: the lanes' 128-bit reads do not collide
    float* q_s = pa_sm;                 // [PA_QT][hs], already divided by sqrt(hs)
    float* k_s = q_s + PA_QT * hs;      // [PA_KT][hs + 4]
    float* v_s = k_s + PA_KT * ks;      // [PA_KT][hs]
    float* p_s = v_s + PA_KT * hs;      // [PA_QT][PA_KT]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.x, t0 = blockIdx.y * PA_QT;
    const int nq = min(PA_QT, n_tokens - t0);
    const int kvh = head / kv_mul;
    const T* kbase = kc + (long long)kvh * head_stride;
    const T* vbase = vc + (long long)kvh * head_stride;
    const float inv = 1.0f / sqrtf((float)hs);
    for (int i = tid; i < PA_QT * hs; i += PA_THREADS) {
        const int tq = i / hs, d = i - tq * hs;
        q_s[i] = tq < nq ? q[(size_t)(t0 + tq) * q_ld + (size_t)head * hs + d] * inv : 0.f;
    }
    float m[4], l[4], acc[4][PA_MAXC][4];
#pragma unroll
    for (int qi = 0; qi < 4; qi++) {
        m[qi] = -INFINITY;
        l[qi] = 0.f;
#pragma unroll
        for (int c = 0; c < PA_MAXC; c++) acc[qi][c][0] = acc[qi][c][1] = acc[qi][c][2] = acc[qi][c][3] = 0.f;
    }
    const int last_pos = pos0 + t0 + nq - 1;           // last position any query of this tile attends to
    const int warp_last = pos0 + t0 + 4 * warp + 3;    // ... any query of this warp
    for (int kt0 = 0; kt0 <= last_pos; kt0 += PA_KT) {
        const int cnt = min(PA_KT, last_pos + 1 - kt0);
        __syncthreads();  // the previous tile has been consumed (and, the first time round, q_s is complete)
        pa_load_rows<T>(kbase + (long long)kt0 * hs, hs, cnt, hs, k_s, ks, tid);
        pa_load_rows<T>(vbase + (long long)kt0 * hs, hs, cnt, hs, v_s, hs, tid);
        __syncthreads();
        if (kt0 > warp_last || 4 * warp >= nq) continue;  // nothing in this tile for this warp's queries (warp-uniform)
        float sc[4] = {0.f, 0.f, 0.f, 0.f};
        const float* kr = k_s + lane * ks;
        const float* qr = q_s + 4 * warp * hs;
        for (int d = 0; d < hs; d += 4) {
            const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
            for (int qi = 0; qi < 4; qi++) {
                const float4 qv = *reinterpret_cast<const float4*>(qr + qi * hs + d);
                sc[qi] = fmaf(kv.x, qv.x, fmaf(kv.y, qv.y, fmaf(kv.z, qv.z, fmaf(kv.w, qv.w, sc[qi]))));
            }
        }
#pragma unroll
        for (int qi = 0; qi < 4; qi++) {
            const int qpos = pos0 + t0 + 4 * warp + qi;
            const bool valid = lane < cnt && kt0 + lane <= qpos && 4 * warp + qi < nq;
            const float sv = valid ? sc[qi] : -INFINITY;
            float mt = sv;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
            const float m_new = fmaxf(m[qi], mt);
            const float pv = valid ? expf(sv - m_new) : 0.f;
            float ps = pv;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            const float resc = m[qi] == -INFINITY ? 0.f : expf(m[qi] - m_new);  // nothing accumulated yet: acc and l are zero anyway
            l[qi] = l[qi] * resc + ps;
            m[qi] = m_new;
#pragma unroll
            for (int c = 0; c < PA_MAXC; c++) {
                acc[qi][c][0] *= resc; acc[qi][c][1] *= resc; acc[qi][c][2] *= resc; acc[qi][c][3] *= resc;
            }
            p_s[(4 * warp + qi) * PA_KT + lane] = pv;
        }
        __syncwarp();
        const float* pr = p_s + 4 * warp * PA_KT;
        for (int j = 0; j < cnt; j += 4) {
            float4 pq[4];
#pragma unroll
            for (int qi = 0; qi < 4; qi++) pq[qi] = *reinterpret_cast<const float4*>(pr + qi * PA_KT + j);
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
#pragma unroll
                for (int c = 0; c < PA_MAXC; c++) {
                    const int d = 128 * c + 4 * lane;
                    if (d < hs) {
                        const float4 vv = *reinterpret_cast<const float4*>(v_s + (size_t)(j + jj) * hs + d);  // rows >= cnt are zero
#pragma unroll
                        for (int qi = 0; qi < 4; qi++) {
                            const float pw = jj == 0 ? pq[qi].x : jj == 1 ? pq[qi].y : jj == 2 ? pq[qi].z : pq[qi].w;
                            acc[qi][c][0] = fmaf(pw, vv.x, acc[qi][c][0]);
                            acc[qi][c][1] = fmaf(pw, vv.y, acc[qi][c][1]);
                            acc[qi][c][2] = fmaf(pw, vv.z, acc[qi][c][2]);
                            acc[qi][c][3] = fmaf(pw, vv.w, acc[qi][c][3]);
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int qi = 0; qi < 4; qi++) {
        const int tq = 4 * warp + qi;
        if (tq < nq) {
#pragma unroll
            for (int c = 0; c < PA_MAXC; c++) {
                const int d = 128 * c + 4 * lane;
                if (d < hs) {
                    const float il = 1.0f / l[qi];  // position 0 is always attended to: l > 0
                    *reinterpret_cast<float4*>(out + (size_t)(t0 + tq) * out_ld + (size_t)head * hs + d) =
                        make_float4(acc[qi][c][0] * il, acc[qi][c][1] * il, acc[qi][c][2] * il, acc[qi][c][3] * il);
                }
            }
        }
    }
}

// ---- small kernels around the GEMMs ---------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum256(float x, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = x;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += sh[w];
    return t;
}
__device__ __forceinline__ void store_hi_lo(__half* hi, __half* lo, size_t i, float y) {
    const __half h = __float2half_rn(y);
    hi[i] = h;
    lo[i] = __float2half_rn(y - __half2float(h));
}

// Row t of X (optionally RmsNorm'd: ops/rms_norm.rs:68-77) as fp16 hi / lo planes [T_pad][K].
__global__ void prefill_split_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ norm_w, float eps, int K,
                                     __half* __restrict__ hi, __half* __restrict__ lo) {
    __shared__ float sh[32];
    const int t = blockIdx.x;
    const float* xr = x + (size_t)t * ldx;
    float mul = 1.f;
    if (norm_w) {
        float s = 0.f;
        for (int i = threadIdx.x; i < K; i += blockDim.x) s += xr[i] * xr[i];
        s = block_sum256(s, sh);
        mul = 1.0f / sqrtf(s / (float)K + eps);
    }
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
        const float y = norm_w ? __fmul_rn(__fmul_rn(xr[i], mul), norm_w[i]) : xr[i];
        store_hi_lo(hi, lo, (size_t)t * K + i, y);
    }
}

// Row t of X after LayerNorm with gamma / beta (ops/layernorm.rs:104-111 and the caller's scale and shift,
// models/gpt2/cpu.rs:239-240) as fp16 hi / lo planes [T_pad][K]; same arithmetic as the decode step's fused prologue.
__global__ void prefill_split_ln_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                                        int K, __half* __restrict__ hi, __half* __restrict__ lo) {
    __shared__ float sh[32];
    const int t = blockIdx.x;
    const float* xr = x + (size_t)t * ldx;
    float s = 0.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) s += xr[i];
    const float mean = block_sum256(s, sh) / (float)K;
    float v = 0.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
        const float d = xr[i] - mean;
        v += d * d;
    }
    v = block_sum256(v, sh);
    const float mul = 1.0f / sqrtf(v / (float)K + eps);
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
        float y = __fmul_rn(__fmul_rn(xr[i] - mean, mul), gamma[i]);
        if (beta) y += beta[i];
        store_hi_lo(hi, lo, (size_t)t * K + i, y);
    }
}

// gelu (ops/unary.rs:81-85) of [T][H] straight into the hi / lo planes of the next GEMM's input.
__global__ void prefill_gelu_split_kernel(const float* __restrict__ g, int H, __half* __restrict__ hi, __half* __restrict__ lo) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= H) return;
    const float x = g[(size_t)t * H + i];
    const float A = 0.044715f, Sq = 0.7978846f;
    store_hi_lo(hi, lo, (size_t)t * H + i, 0.5f * x * (1.0f + tanhf(Sq * x * (1.0f + A * x * x))));
}

// x[t] += row (pos0 + t) of a table of position vectors (models/gpt2/cpu.rs:227-228).
__global__ void prefill_add_rows_kernel(float* __restrict__ x, int dim, const float* __restrict__ table, int pos0) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < dim) x[(size_t)t * dim + i] += table[(size_t)(pos0 + t) * dim + i];
}

// hb = up * gate / (1 + exp(-gate)) (ops/silu.rs:50-58) straight into the hi / lo planes of the down projection's input.
__global__ void prefill_silu_split_kernel(const float* __restrict__ gate, const float* __restrict__ up, int H, __half* __restrict__ hi,
                                          __half* __restrict__ lo) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= H) return;
    const float g = gate[(size_t)t * H + i], u = up[(size_t)t * H + i];
    store_hi_lo(hi, lo, (size_t)t * H + i, u * (g / (1.0f + expf(-g))));
}

// x[t] = row token[t] of the embedding table (f32 table or quantised matrix).
__global__ void prefill_embed_kernel(float* __restrict__ x, int dim, const int* __restrict__ tokens, const float* __restrict__ table,
                                     int fmt, const uint8_t* __restrict__ qdata) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim) return;
    const long long row = tokens[t];
    x[(size_t)t * dim + i] = table ? table[row * dim + i] : dequant_elem(fmt, qdata, dim, row, i);
}

// RoPE (ops/rope.rs:88-125; both variants) on q and k of token t at position pos0 + t (or *d_pos + t), q to `q_out`
// (may be its source), k and, when given, v into the cache ([kv_head][position][head_size], f16 or f32): the q/k/v
// epilogue of the decode step for T tokens at once, and the decode step's own RoPE stage where the fused epilogue
// cannot serve (pairs half a head apart, dense f32 matrices).
__global__ void rope_kv_store_kernel(const float* __restrict__ q_src, const float* __restrict__ k_src, const float* __restrict__ v_src,
                                     int ld, int q_dim, int kv_dim, int head_size, int pos0, const int* __restrict__ d_pos,
                                     const float* __restrict__ theta, int neox, float* __restrict__ q_out, int ldq, void* kcache, void* vcache,
                                     int kv_f16, long long kv_head_stride, long long seq_stride) {
    const int t = blockIdx.y;
    const int p = blockIdx.x * blockDim.x + threadIdx.x;  // pair index over q then k; then plain copies of v
    // seq_stride > 0: row t is a sequence of its own, at position d_pos[t] of caches seq_stride bytes after row t - 1's
    const int pos = seq_stride > 0 ? d_pos[t] : (d_pos ? *d_pos : pos0) + t;
    if (pos < 0) return;
    kcache = reinterpret_cast<char*>(kcache) + (size_t)t * seq_stride;
    vcache = reinterpret_cast<char*>(vcache) + (size_t)t * seq_stride;
    const int nq = q_dim / 2, nk = kv_dim / 2;
    if (p < nq + nk) {
        const bool is_k = p >= nq;
        const int i = is_k ? p - nq : p;
        const float* src = (is_k ? k_src : q_src) + (size_t)t * ld;
        const int head = (2 * i) / head_size, fi = ((2 * i) % head_size) >> 1;
        int a, b;
        if (neox) {
            a = head * head_size + fi;
            b = a + head_size / 2;
        } else {
            a = 2 * i;
            b = a + 1;
        }
        float sn, cs;
        sincosf((float)pos * theta[fi], &sn, &cs);
        const float xa = src[a], xb = src[b];
        const float ya = cs * xa - sn * xb, yb = sn * xa + cs * xb;
        if (!is_k) {
            q_out[(size_t)t * ldq + a] = ya;
            q_out[(size_t)t * ldq + b] = yb;
        } else {
            const int ha = a / head_size, da = a % head_size, hb = b / head_size, db = b % head_size;
            const long long oa = (long long)pos * head_size + ha * kv_head_stride + da, ob = (long long)pos * head_size + hb * kv_head_stride + db;
            if (kv_f16) {
                reinterpret_cast<__half*>(kcache)[oa] = __float2half_rn(ya);
                reinterpret_cast<__half*>(kcache)[ob] = __float2half_rn(yb);
            } else {
                reinterpret_cast<float*>(kcache)[oa] = ya;
                reinterpret_cast<float*>(kcache)[ob] = yb;
            }
        }
    } else if (v_src && p < nq + nk + kv_dim) {
        const int e = p - nq - nk;
        const float y = v_src[(size_t)t * ld + e];
        const long long o = (long long)pos * head_size + (e / head_size) * kv_head_stride + e % head_size;
        if (kv_f16) reinterpret_cast<__half*>(vcache)[o] = __float2half_rn(y);
        else reinterpret_cast<float*>(vcache)[o] = y;
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// fp16 plane [rows][K] row-major -> boxes of 64 columns x `box_rows` rows, 128-byte swizzle (what umma_desc describes).
int make_plane_map(slai_ctx* ctx, CUtensorMap* map, const __half* base, int rows, int K, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    SLAI_REQUIRE(ctx, enc, SLAI_ERR_CUDA, "prefill: the driver does not provide cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)PF_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SLAI_REQUIRE(ctx, r == CUDA_SUCCESS, SLAI_ERR_CUDA, "prefill: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return SLAI_OK;
}

}  // namespace

size_t prefill_gemm_smem(int NT) { return (size_t)PF_STAGES * (2 * PF_A_BYTES + 2 * (size_t)NT * PF_BK * 2) + 1024; }

// Y[t][out_off + m] = (resid[t][m] +) sum_k W[m][k] X[t][k] (+ bias[m]) for t < T, with X given as hi / lo planes of
// `t_pad` rows (a multiple of NT; rows >= T are zero).
int prefill_gemm_launch(slai_ctx* ctx, const PrefillGemm& G) {
    const slai_qmatrix* w = G.w;
    SLAI_REQUIRE(ctx, w->fmt == SLAI_FMT_Q4_K || w->fmt == SLAI_FMT_Q5_K || w->fmt == SLAI_FMT_Q6_K || w->fmt == SLAI_FMT_Q8_0,
                 SLAI_ERR_UNSUPPORTED_FORMAT, "prefill: format %d has no GEMM path", w->fmt);
    SLAI_REQUIRE(ctx, w->ncols % PF_BK == 0 && G.NT % 16 == 0 && G.NT >= 16 && G.NT <= 256 && G.t_pad % G.NT == 0 && G.T <= G.t_pad,
                 SLAI_ERR_SHAPE, "prefill: K=%lld / tile of %d tokens not supported", (long long)w->ncols, G.NT);
    CUtensorMap map_hi, map_lo;
    int rc = make_plane_map(ctx, &map_hi, G.x_hi, G.t_pad, (int)w->ncols, G.NT);
    if (rc) return rc;
    if ((rc = make_plane_map(ctx, &map_lo, G.x_lo, G.t_pad, (int)w->ncols, G.NT))) return rc;
    PrefillGemmParams P;
    P.w = w->data; P.tile_bytes = w->tile_bytes; P.fmt = w->fmt; P.M = G.rows; P.K = (int)w->ncols;
    P.T = G.T; P.NT = G.NT; P.out = G.out; P.ldo = G.ldo; P.out_off = G.out_off; P.resid = G.resid; P.ldr = G.ldr; P.bias = G.bias;
    P.err_flag = ctx->d_counters + CNT_ERR_FLAG;
    P.wait_limit = ctx->wait_limit;
    const size_t smem = prefill_gemm_smem(G.NT);
    static PerDeviceOnce attr;
    if (attr.need(ctx->device)) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(prefill_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_gemm_smem(256)));
        attr.set(ctx->device);
    }
    const dim3 grid((unsigned)((G.rows + PF_BM - 1) / PF_BM), (unsigned)(G.t_pad / G.NT));
    prefill_gemm_kernel<<<grid, PF_THREADS, smem, ctx->stream>>>(P, map_hi, map_lo);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}

int prefill_split_launch(slai_ctx* ctx, const float* x, int ldx, const float* norm_w, float eps, int T, int K, __half* hi, __half* lo) {
    prefill_split_kernel<<<T, 256, 0, ctx->stream>>>(x, ldx, norm_w, eps, K, hi, lo);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
int prefill_split_ln_launch(slai_ctx* ctx, const float* x, int ldx, const float* gamma, const float* beta, float eps, int T, int K, __half* hi,
                            __half* lo) {
    prefill_split_ln_kernel<<<T, 256, 0, ctx->stream>>>(x, ldx, gamma, beta, eps, K, hi, lo);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
int prefill_gelu_split_launch(slai_ctx* ctx, const float* g, int T, int H, __half* hi, __half* lo) {
    prefill_gelu_split_kernel<<<dim3((H + 255) / 256, T), 256, 0, ctx->stream>>>(g, H, hi, lo);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
int prefill_add_rows_launch(slai_ctx* ctx, float* x, int dim, const float* table, int pos0, int T) {
    prefill_add_rows_kernel<<<dim3((dim + 255) / 256, T), 256, 0, ctx->stream>>>(x, dim, table, pos0);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
int prefill_silu_split_launch(slai_ctx* ctx, const float* gate, const float* up, int T, int H, __half* hi, __half* lo) {
    prefill_silu_split_kernel<<<dim3((H + 255) / 256, T), 256, 0, ctx->stream>>>(gate, up, H, hi, lo);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
int prefill_embed_launch(slai_ctx* ctx, float* x, int dim, const int* d_tokens, int T, const float* table, const slai_qmatrix* qtable) {
    prefill_embed_kernel<<<dim3((dim + 255) / 256, T), 256, 0, ctx->stream>>>(x, dim, d_tokens, table, qtable ? qtable->fmt : 0,
                                                                             qtable ? qtable->data : nullptr);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
// Causal attention of prompt tokens pos0 .. pos0 + T - 1 over the caches (which already hold their keys and values).
// Returns SLAI_ERR_UNSUPPORTED_FORMAT for head sizes the kernel does not take (the caller then uses the decode kernel).
bool prefill_attention_supported(int head_size, int kv_f16, const void* kc, const void* vc, long long head_stride) {
    const int esz = kv_f16 ? 2 : 4;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc) | (uintptr_t)(head_stride * esz) | (uintptr_t)(head_size * esz);
    return head_size % 8 == 0 && head_size <= 128 * PA_MAXC && (bits & 15) == 0;
}
int prefill_attention_launch(slai_ctx* ctx, const float* q, int q_ld, const void* kc, const void* vc, int kv_f16, long long head_stride, int head_size,
                             int n_heads, int kv_mul, int pos0, int T, float* out, int out_ld) {
    SLAI_REQUIRE(ctx, prefill_attention_supported(head_size, kv_f16, kc, vc, head_stride) && q_ld % 4 == 0 && out_ld % 4 == 0, SLAI_ERR_UNSUPPORTED_FORMAT,
                 "prefill attention: head size %d / alignment not supported", head_size);
    const size_t smem = ((size_t)PA_QT * head_size + (size_t)PA_KT * (head_size + 4) + (size_t)PA_KT * head_size + PA_QT * PA_KT) * 4;
    const dim3 grid((unsigned)n_heads, (unsigned)((T + PA_QT - 1) / PA_QT));
    static PerDeviceOnce attr;
    if (attr.need(ctx->device)) {
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(prefill_attn_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        SLAI_CHECK_CUDA(ctx, cudaFuncSetAttribute(prefill_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        attr.set(ctx->device);
    }
    if (kv_f16)
        prefill_attn_kernel<__half><<<grid, PA_THREADS, smem, ctx->stream>>>(q, q_ld, (const __half*)kc, (const __half*)vc, head_stride, head_size, kv_mul, pos0, T, out, out_ld);
    else
        prefill_attn_kernel<float><<<grid, PA_THREADS, smem, ctx->stream>>>(q, q_ld, (const float*)kc, (const float*)vc, head_stride, head_size, kv_mul, pos0, T, out, out_ld);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
int prefill_rope_kv_launch(slai_ctx* ctx, const float* qkv, int ld, int q_dim, int kv_dim, int head_size, int pos0, int T,
                           const float* theta, int neox, float* q_out, void* kcache, void* vcache, int kv_f16, long long kv_head_stride) {
    const int work = q_dim / 2 + kv_dim / 2 + kv_dim;
    rope_kv_store_kernel<<<dim3((work + 255) / 256, T), 256, 0, ctx->stream>>>(qkv, qkv + q_dim, qkv + q_dim + kv_dim, ld, q_dim, kv_dim, head_size,
                                                                              pos0, nullptr, theta, neox, q_out, q_dim, kcache, vcache, kv_f16,
                                                                              kv_head_stride, 0);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
// One token at the device-side position: q rotated in place, k (and v when given) into the cache.
int rope_kv_store_launch(slai_ctx* ctx, float* q, const float* k, const float* v, int q_dim, int kv_dim, int head_size, const int* d_pos,
                         const float* theta, int neox, void* kcache, void* vcache, int kv_f16, long long kv_head_stride, bool pdl) {
    const int work = q_dim / 2 + kv_dim / 2 + (v ? kv_dim : 0);
    (void)pdl;
    rope_kv_store_kernel<<<dim3((work + 255) / 256, 1), 256, 0, ctx->stream>>>(q, k, v, 0, q_dim, kv_dim, head_size, 0, d_pos, theta, neox, q, q_dim,
                                                                              kcache, vcache, kv_f16, kv_head_stride, 0);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
int rope_kv_store_seqs_launch(slai_ctx* ctx, const float* qkv, int ld, int q_dim, int kv_dim, int head_size, const int* d_pos, int B,
                              const float* theta, int neox, float* q_out, void* kcache, void* vcache, int kv_f16, long long kv_head_stride,
                              long long seq_stride) {
    SLAI_REQUIRE(ctx, seq_stride > 0 && d_pos && B >= 1, SLAI_ERR_INVALID_ARG, "rope: a batch of sequences needs positions and a cache stride");
    const int work = q_dim / 2 + kv_dim / 2 + kv_dim;
    rope_kv_store_kernel<<<dim3((work + 255) / 256, B), 256, 0, ctx->stream>>>(qkv, qkv + q_dim, qkv + q_dim + kv_dim, ld, q_dim, kv_dim, head_size,
                                                                              0, d_pos, theta, neox, q_out, q_dim, kcache, vcache, kv_f16,
                                                                              kv_head_stride, seq_stride);
    SLAI_CHECK_CUDA(ctx, cudaGetLastError());
    return SLAI_OK;
}
