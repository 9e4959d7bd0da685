// Per-format MMA bodies of the dequant-GEMV kernel (see gemv.cu for the kernel shape, layout.cuh for the
// tile-step blocks they read from shared memory and gemv_frag.cuh for the operand mapping).  The functions
// are written against a small set of primitives (shared loads, the integer m16n8k32 MMA) that have a device
// implementation in PTX and a host implementation in which 32 CPU threads play the lanes of a warp, so the
// very same source is exercised by the CPU test-suite (tests/host_emul.cpp) before it ever runs on a GPU.
#pragma once
#include "gemv_frag.cuh"

#ifndef __CUDA_ARCH__
#include <pthread.h>
#include <string.h>
namespace hostemu {
// One emulated warp: 32 host threads, a barrier, an exchange area for MMA operands, and a byte array that
// stands for shared memory (shared-space addresses are offsets into it).
struct Warp {
    pthread_barrier_t bar;
    uint32_t a[32][4], b[32][2];
    unsigned char* smem;
};
extern thread_local int lane;
extern thread_local Warp* warp;
}  // namespace hostemu
#endif

namespace prim {

SLAI_HD uint4 lds16(uint32_t addr) {
#ifdef __CUDA_ARCH__
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
#else
    uint4 r;
    memcpy(&r, hostemu::warp->smem + addr, 16);
    return r;
#endif
}
SLAI_HD uint32_t lds32(uint32_t addr) {
#ifdef __CUDA_ARCH__
    uint32_t r;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(addr));
    return r;
#else
    uint32_t r;
    memcpy(&r, hostemu::warp->smem + addr, 4);
    return r;
#endif
}
SLAI_HD uint2 lds8(uint32_t addr) {
#ifdef __CUDA_ARCH__
    uint2 r;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(addr));
    return r;
#else
    uint2 r;
    memcpy(&r, hostemu::warp->smem + addr, 8);
    return r;
#endif
}
SLAI_HD uint32_t lds_u16(uint32_t addr) {
#ifdef __CUDA_ARCH__
    unsigned short r;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(r) : "r"(addr));
    return r;
#else
    unsigned short r;
    memcpy(&r, hostemu::warp->smem + addr, 2);
    return r;
#endif
}
SLAI_HD float h2f(uint32_t bits16) {
#ifdef __CUDA_ARCH__
    return __half2float(__ushort_as_half((unsigned short)bits16));
#else
    __half_raw hr;
    hr.x = (unsigned short)bits16;
    return __half2float(__half(hr));
#endif
}
SLAI_HD float fma(float a, float b, float c) {
#ifdef __CUDA_ARCH__
    return fmaf(a, b, c);
#else
    return (float)((double)a * (double)b + (double)c);  // single rounding, like fmaf
#endif
}
// D = A(16x32, row) * B(32x8, col, s8) + D (s32); A holds s8 or (UA) u8 values.  Lane (g = lane/4, t = lane%4):
//   a0 = A[g][4t..4t+3], a1 = A[g+8][4t..], a2 = A[g][16+4t..], a3 = A[g+8][16+4t..]   (4 x 8 bit per register)
//   b0 = B[4t..4t+3][g], b1 = B[16+4t..][g];   c0,c1 = D[g][2t..2t+1], c2,c3 = D[g+8][2t..2t+1]
// ZERO: D = A * B (the accumulator input is the constant zero, no registers are cleared first).
template <bool UA, bool ZERO>
SLAI_HD void mma_i8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
#ifdef __CUDA_ARCH__
    if (ZERO) {
        if (UA)
            asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
        else
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    } else {
        if (UA)
            asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
        else
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
#else
    hostemu::Warp* W = hostemu::warp;
    const int lane = hostemu::lane;
    W->a[lane][0] = a0; W->a[lane][1] = a1; W->a[lane][2] = a2; W->a[lane][3] = a3;
    W->b[lane][0] = b0; W->b[lane][1] = b1;
    pthread_barrier_wait(&W->bar);
    auto A = [&](int row, int k) {
        const int l = (row & 7) * 4 + ((k & 15) >> 2);
        const int reg = (row >= 8 ? 1 : 0) + (k >= 16 ? 2 : 0);
        const uint32_t byte = (W->a[l][reg] >> (8 * (k & 3))) & 0xFF;
        return UA ? (int)byte : (int)(signed char)byte;
    };
    auto B = [&](int k, int n) {
        const int l = n * 4 + ((k & 15) >> 2);
        const int reg = k >= 16 ? 1 : 0;
        return (int)(signed char)((W->b[l][reg] >> (8 * (k & 3))) & 0xFF);
    };
    const int g = lane >> 2, t = lane & 3;
    for (int i = 0; i < 4; i++) {
        const int row = g + (i >= 2 ? 8 : 0), col = 2 * t + (i & 1);
        int s = ZERO ? 0 : c[i];
        for (int k = 0; k < 32; k++) s += A(row, k) * B(k, col);
        c[i] = s;
    }
    pthread_barrier_wait(&W->bar);
#endif
}

}  // namespace prim

namespace gemvfmt {

using namespace frag;

// Shared-space byte addresses of the staged activation vector:
//   dig   four planes of s8 digits (plane p at dig + p*plane, element k at byte k)
//   sv    per-sub-block digit sums: Q6_K 4 x s32 per 16 elements; Q4_K / Q5_K a byte table for the tensor
//         cores, per 256-element step eight rows (digit plane q, part: row 2q = high, 2q+1 = low base-128 digit of
//         the sum) of 16 bytes: byte j = sub-block j of the step, bytes 8..15 zero
//   zero  256 zero bytes: lanes whose B column belongs to the other sub-block read their operand here
struct Smem {
    uint32_t dig, plane, sv, zero;
};
constexpr int ZERO_BYTES = 256;

struct LaneCtx {
    int lane, g, t;
    uint32_t bbase;   // this lane's B operand of step s, sub-block offset o is at bbase + s * bmul + o
    uint32_t bmul;    // bytes of digits per step (0 for lanes that read zeros)
    float wd0, wd1;   // weights of the two digits whose sums this lane holds (digits 2(t&1), 2(t&1)+1)
    float wq;         // weight of digit plane t (Q4_K / Q5_K: the lane holds that plane's sum for the minimum term)
};

// F::BOFF(t): byte offset inside a step's digits of the first operand of lane t; F::STEP digits per step;
// F::PRESCALE: factor the integer sums carry (folded into the digit weights).
template <class F>
SLAI_HD void lane_init(LaneCtx& L, int lane, const Smem& S) {
    L.lane = lane;
    L.g = lane >> 2;
    L.t = lane & 3;
    const bool bact = (L.t >> 1) == (L.g >> 2);  // the lane's column belongs to its own sub-block
    L.bbase = bact ? S.dig + (L.g & 3) * S.plane + F::boff(L.t) : S.zero;
    L.bmul = bact ? F::STEP : 0;
    L.wd0 = digit_weight(2 * (L.t & 1)) * F::PRESCALE;
    L.wd1 = digit_weight(2 * (L.t & 1) + 1) * F::PRESCALE;
    L.wq = digit_weight(L.t);
}

SLAI_HD float combine(int p0, int p1, const LaneCtx& L) { return prim::fma((float)p1, L.wd1, (float)p0 * L.wd0); }
SLAI_HD uint32_t byte_of(uint32_t w, int i) {
#ifdef __CUDA_ARCH__
    return __byte_perm(w, 0u, 0x4440u | (uint32_t)i);  // one instruction
#else
    return (w >> (8 * i)) & 0xFFu;
#endif
}

// Every format provides
//   STEP      elements of K per tile-step block          SV_GRAN  elements per digit-sum entry (0: none)
//   compute   one tile-step block at shared address `blk` (K step number `step`): accumulates rows g and g+8
// ---- Q4_K / Q5_K ---------------------------------------------------------------------------
// Block header (layout.cuh): row r at 20 r = { f16 d, f16 dmin, u8 sc[8] in lane order, u8 m[8] }.
//  * main term: per (ci, nib) two MMAs give the lane the sums of its own sub-block for two digits; they are
//    multiplied by the sub-block's 6-bit scale and added up in integers.  Q4_K feeds the high nibbles unshifted
//    (16 q as u8) and multiplies the low-nibble scales by 16 instead: every sum carries the factor 16.
//  * minimum term: sum_j m[r][j] * S_j (S_j = digit sums of sub-block j) is one more MMA per step: A = the m bytes
//    of the 16 rows, B = the byte table of the sums; lane t ends up with the sum for digit plane t.
template <bool FIVE>
struct K45 {
    static constexpr int FMT = FIVE ? 13 : 12;
    static constexpr int STEP_BYTES = FIVE ? 2880 : 2368;
    static constexpr int STEP = 256;
    static constexpr int SV_GRAN = 32;
    static constexpr float PRESCALE = FIVE ? 1.0f : 0.0625f;
    static constexpr int QOFF = FIVE ? 320 + 512 : 320;
    SLAI_HD static uint32_t boff(int t) { return 64 * (t >> 1) + 16 * (t & 1); }
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const uint32_t hA = blk + 20 * L.g, hB = hA + 160;
        const uint32_t ddA = prim::lds32(hA), ddB = prim::lds32(hB);
        const uint32_t scA = prim::lds32(hA + 4 + 4 * (L.t >> 1)), scB = prim::lds32(hB + 4 + 4 * (L.t >> 1));
        const uint32_t mA = prim::lds32(hA + 12 + 4 * (L.t & 1)), mB = prim::lds32(hB + 12 + 4 * (L.t & 1));
        const uint32_t bq = prim::lds32(S.sv + 128 * step + 16 * L.g + 4 * L.t);
        int cq[4];
        prim::mma_i8<true, true>(cq, mA, mB, 0u, 0u, bq, 0u);
        uint4 hqA = make_uint4(0u, 0u, 0u, 0u), hqB = hqA;
        if (FIVE) {
            hqA = prim::lds16(blk + 320 + 32 * L.g + 16 * (L.t & 1));
            hqB = prim::lds16(blk + 320 + 32 * (L.g + 8) + 16 * (L.t & 1));
        }
        const uint32_t q0 = blk + QOFF + 16 * L.lane;
        const uint32_t ba = L.bbase + (uint32_t)step * L.bmul;
        int PA0 = 0, PA1 = 0, PB0 = 0, PB1 = 0;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint4 qA = prim::lds16(q0 + (ci * 2) * 512), qB = prim::lds16(q0 + (ci * 2 + 1) * 512);
            const int hsh = 2 * ((L.t >> 1) + 2 * ci);  // Q5_K: 2 * (64-element group index)
            const uint32_t hAx = hqA.x >> hsh, hAy = hqA.y >> hsh, hAz = hqA.z >> hsh, hAw = hqA.w >> hsh;
            const uint32_t hBx = hqB.x >> hsh, hBy = hqB.y >> hsh, hBz = hqB.z >> hsh, hBw = hqB.w >> hsh;
#pragma unroll
            for (int nib = 0; nib < 2; nib++) {
                // sub-block 4 ci + 2 (t >> 1) + nib of the step
                const uint4 bv = prim::lds16(ba + 128 * ci + 32 * nib);
                int c[4];
                uint32_t sA = byte_of(scA, 2 * ci + nib), sB = byte_of(scB, 2 * ci + nib);
                if (FIVE) {
                    prim::mma_i8<true, true>(c, q5_nibs(qA.x, hAx, nib), q5_nibs(qB.x, hBx, nib), q5_nibs(qA.y, hAy, nib), q5_nibs(qB.y, hBy, nib), bv.x, bv.y);
                    prim::mma_i8<true, false>(c, q5_nibs(qA.z, hAz, nib), q5_nibs(qB.z, hBz, nib), q5_nibs(qA.w, hAw, nib), q5_nibs(qB.w, hBw, nib), bv.z, bv.w);
                } else {
                    const uint32_t mk = nib ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
                    prim::mma_i8<true, true>(c, qA.x & mk, qB.x & mk, qA.y & mk, qB.y & mk, bv.x, bv.y);
                    prim::mma_i8<true, false>(c, qA.z & mk, qB.z & mk, qA.w & mk, qB.w & mk, bv.z, bv.w);
                    if (nib == 0) {
                        sA <<= 4;
                        sB <<= 4;
                    }
                }
                PA0 += (int)sA * c[0]; PA1 += (int)sA * c[1];
                PB0 += (int)sB * c[2]; PB1 += (int)sB * c[3];
            }
        }
        const float dA = prim::h2f(ddA & 0xFFFF), mnA = prim::h2f(ddA >> 16);
        const float dB = prim::h2f(ddB & 0xFFFF), mnB = prim::h2f(ddB >> 16);
        accA = prim::fma(dA, combine(PA0, PA1, L), accA);
        accA = prim::fma(-mnA, (float)(cq[0] * 128 + cq[1]) * L.wq, accA);
        accB = prim::fma(dB, combine(PB0, PB1, L), accB);
        accB = prim::fma(-mnB, (float)(cq[2] * 128 + cq[3]) * L.wq, accB);
    }
    // The same step against NV staged vectors at once (vector v's digits `bvs` bytes after vector v-1's for the lanes that
    // read digits, its sum table `svs` bytes after): the packed weights are loaded and masked once, every vector adds its
    // own MMAs.  Per vector the arithmetic, and its order, is that of `compute`.
    template <int NV>
    SLAI_HD static void compute_batch(uint32_t blk, int step, const LaneCtx& L, const Smem& S, uint32_t bvs, uint32_t svs, float (&accA)[NV],
                                      float (&accB)[NV]) {
        const uint32_t hA = blk + 20 * L.g, hB = hA + 160;
        const uint32_t ddA = prim::lds32(hA), ddB = prim::lds32(hB);
        const uint32_t scA = prim::lds32(hA + 4 + 4 * (L.t >> 1)), scB = prim::lds32(hB + 4 + 4 * (L.t >> 1));
        const uint32_t mA = prim::lds32(hA + 12 + 4 * (L.t & 1)), mB = prim::lds32(hB + 12 + 4 * (L.t & 1));
        uint4 hqA = make_uint4(0u, 0u, 0u, 0u), hqB = hqA;
        if (FIVE) {
            hqA = prim::lds16(blk + 320 + 32 * L.g + 16 * (L.t & 1));
            hqB = prim::lds16(blk + 320 + 32 * (L.g + 8) + 16 * (L.t & 1));
        }
        const uint32_t q0 = blk + QOFF + 16 * L.lane;
        const uint32_t ba = L.bbase + (uint32_t)step * L.bmul;
        int PA0[NV], PA1[NV], PB0[NV], PB1[NV];
#pragma unroll
        for (int v = 0; v < NV; v++) PA0[v] = PA1[v] = PB0[v] = PB1[v] = 0;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint4 qA = prim::lds16(q0 + (ci * 2) * 512), qB = prim::lds16(q0 + (ci * 2 + 1) * 512);
            const int hsh = 2 * ((L.t >> 1) + 2 * ci);
            const uint32_t hAx = hqA.x >> hsh, hAy = hqA.y >> hsh, hAz = hqA.z >> hsh, hAw = hqA.w >> hsh;
            const uint32_t hBx = hqB.x >> hsh, hBy = hqB.y >> hsh, hBz = hqB.z >> hsh, hBw = hqB.w >> hsh;
#pragma unroll
            for (int nib = 0; nib < 2; nib++) {
                uint32_t sA = byte_of(scA, 2 * ci + nib), sB = byte_of(scB, 2 * ci + nib);
                uint32_t a[8];
                if (FIVE) {
                    a[0] = q5_nibs(qA.x, hAx, nib); a[1] = q5_nibs(qB.x, hBx, nib); a[2] = q5_nibs(qA.y, hAy, nib); a[3] = q5_nibs(qB.y, hBy, nib);
                    a[4] = q5_nibs(qA.z, hAz, nib); a[5] = q5_nibs(qB.z, hBz, nib); a[6] = q5_nibs(qA.w, hAw, nib); a[7] = q5_nibs(qB.w, hBw, nib);
                } else {
                    const uint32_t mk = nib ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
                    a[0] = qA.x & mk; a[1] = qB.x & mk; a[2] = qA.y & mk; a[3] = qB.y & mk;
                    a[4] = qA.z & mk; a[5] = qB.z & mk; a[6] = qA.w & mk; a[7] = qB.w & mk;
                    if (nib == 0) {
                        sA <<= 4;
                        sB <<= 4;
                    }
                }
#pragma unroll
                for (int v = 0; v < NV; v++) {
                    const uint4 bv = prim::lds16(ba + (uint32_t)v * bvs + 128 * ci + 32 * nib);
                    int c[4];
                    prim::mma_i8<true, true>(c, a[0], a[1], a[2], a[3], bv.x, bv.y);
                    prim::mma_i8<true, false>(c, a[4], a[5], a[6], a[7], bv.z, bv.w);
                    PA0[v] += (int)sA * c[0]; PA1[v] += (int)sA * c[1];
                    PB0[v] += (int)sB * c[2]; PB1[v] += (int)sB * c[3];
                }
            }
        }
        const float dA = prim::h2f(ddA & 0xFFFF), mnA = prim::h2f(ddA >> 16);
        const float dB = prim::h2f(ddB & 0xFFFF), mnB = prim::h2f(ddB >> 16);
#pragma unroll
        for (int v = 0; v < NV; v++) {
            const uint32_t bq = prim::lds32(S.sv + (uint32_t)v * svs + 128 * step + 16 * L.g + 4 * L.t);
            int cq[4];
            prim::mma_i8<true, true>(cq, mA, mB, 0u, 0u, bq, 0u);
            accA[v] = prim::fma(dA, combine(PA0[v], PA1[v], L), accA[v]);
            accA[v] = prim::fma(-mnA, (float)(cq[0] * 128 + cq[1]) * L.wq, accA[v]);
            accB[v] = prim::fma(dB, combine(PB0[v], PB1[v], L), accB[v]);
            accB[v] = prim::fma(-mnB, (float)(cq[2] * 128 + cq[3]) * L.wq, accB[v]);
        }
    }
};
using Q4K = K45<false>;
using Q5K = K45<true>;

// ---- Q6_K ----------------------------------------------------------------------------------
struct Q6K {
    static constexpr int FMT = 14;
    static constexpr int STEP_BYTES = 3360;
    static constexpr int STEP = 256;
    static constexpr int SV_GRAN = 16;
    static constexpr float PRESCALE = 1.0f;
    SLAI_HD static uint32_t boff(int t) { return 16 * (t >> 1) + 8 * (t & 1); }
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        int PA0 = 0, PA1 = 0, PB0 = 0, PB1 = 0;
        const uint32_t ba = L.bbase + (uint32_t)step * L.bmul;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint2 qhA = prim::lds8(blk + 2048 + (h * 2) * 256 + 8 * L.lane), qhB = prim::lds8(blk + 2048 + (h * 2 + 1) * 256 + 8 * L.lane);
            const uint2 scwA = prim::lds8(blk + 3072 + 16 * L.g + 8 * h), scwB = prim::lds8(blk + 3072 + 16 * (L.g + 8) + 8 * h);
#pragma unroll
            for (int pair = 0; pair < 2; pair++) {
                const uint2 qlA = prim::lds8(blk + ((h * 2 + pair) * 2) * 256 + 8 * L.lane);
                const uint2 qlB = prim::lds8(blk + ((h * 2 + pair) * 2 + 1) * 256 + 8 * L.lane);
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    const int sh = 2 * pair + 4 * nib;
                    const int j8 = 4 * nib + 2 * pair + (L.t >> 1);  // sub-block (of 16) inside the half
                    const int j = 16 * step + 8 * h + j8;
                    const uint2 bv = prim::lds8(ba + 128 * h + 64 * nib + 32 * pair);
                    int c[4];
                    prim::mma_i8<false, true>(c, q6_nibs(qlA.x, qhA.x >> sh, nib), q6_nibs(qlB.x, qhB.x >> sh, nib), q6_nibs(qlA.y, qhA.y >> sh, nib),
                                              q6_nibs(qlB.y, qhB.y >> sh, nib), bv.x, bv.y);
                    const uint2 sv = prim::lds8(S.sv + 16 * j + 8 * (L.t & 1));
                    // int8 scale of sub-block j8: byte j8 of the half's 8 scale bytes
                    const uint32_t wsA = j8 < 4 ? scwA.x : scwA.y, wsB = j8 < 4 ? scwB.x : scwB.y;
                    const int scA = (int)(signed char)((wsA >> (8 * (j8 & 3))) & 0xFF), scB = (int)(signed char)((wsB >> (8 * (j8 & 3))) & 0xFF);
                    PA0 += scA * (c[0] - 32 * (int)sv.x); PA1 += scA * (c[1] - 32 * (int)sv.y);
                    PB0 += scB * (c[2] - 32 * (int)sv.x); PB1 += scB * (c[3] - 32 * (int)sv.y);
                }
            }
        }
        const float dA = prim::h2f(prim::lds_u16(blk + 3328 + 2 * L.g)), dB = prim::h2f(prim::lds_u16(blk + 3328 + 2 * (L.g + 8)));
        accA = prim::fma(dA, combine(PA0, PA1, L), accA);
        accB = prim::fma(dB, combine(PB0, PB1, L), accB);
    }
    template <int NV>
    SLAI_HD static void compute_batch(uint32_t blk, int step, const LaneCtx& L, const Smem& S, uint32_t bvs, uint32_t svs, float (&accA)[NV],
                                      float (&accB)[NV]) {
        int PA0[NV], PA1[NV], PB0[NV], PB1[NV];
#pragma unroll
        for (int v = 0; v < NV; v++) PA0[v] = PA1[v] = PB0[v] = PB1[v] = 0;
        const uint32_t ba = L.bbase + (uint32_t)step * L.bmul;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint2 qhA = prim::lds8(blk + 2048 + (h * 2) * 256 + 8 * L.lane), qhB = prim::lds8(blk + 2048 + (h * 2 + 1) * 256 + 8 * L.lane);
            const uint2 scwA = prim::lds8(blk + 3072 + 16 * L.g + 8 * h), scwB = prim::lds8(blk + 3072 + 16 * (L.g + 8) + 8 * h);
#pragma unroll
            for (int pair = 0; pair < 2; pair++) {
                const uint2 qlA = prim::lds8(blk + ((h * 2 + pair) * 2) * 256 + 8 * L.lane);
                const uint2 qlB = prim::lds8(blk + ((h * 2 + pair) * 2 + 1) * 256 + 8 * L.lane);
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    const int sh = 2 * pair + 4 * nib;
                    const int j8 = 4 * nib + 2 * pair + (L.t >> 1);
                    const int j = 16 * step + 8 * h + j8;
                    const uint32_t a0 = q6_nibs(qlA.x, qhA.x >> sh, nib), a1 = q6_nibs(qlB.x, qhB.x >> sh, nib);
                    const uint32_t a2 = q6_nibs(qlA.y, qhA.y >> sh, nib), a3 = q6_nibs(qlB.y, qhB.y >> sh, nib);
                    const uint32_t wsA = j8 < 4 ? scwA.x : scwA.y, wsB = j8 < 4 ? scwB.x : scwB.y;
                    const int scA = (int)(signed char)((wsA >> (8 * (j8 & 3))) & 0xFF), scB = (int)(signed char)((wsB >> (8 * (j8 & 3))) & 0xFF);
#pragma unroll
                    for (int v = 0; v < NV; v++) {
                        const uint2 bv = prim::lds8(ba + (uint32_t)v * bvs + 128 * h + 64 * nib + 32 * pair);
                        int c[4];
                        prim::mma_i8<false, true>(c, a0, a1, a2, a3, bv.x, bv.y);
                        const uint2 sv = prim::lds8(S.sv + (uint32_t)v * svs + 16 * j + 8 * (L.t & 1));
                        PA0[v] += scA * (c[0] - 32 * (int)sv.x); PA1[v] += scA * (c[1] - 32 * (int)sv.y);
                        PB0[v] += scB * (c[2] - 32 * (int)sv.x); PB1[v] += scB * (c[3] - 32 * (int)sv.y);
                    }
                }
            }
        }
        const float dA = prim::h2f(prim::lds_u16(blk + 3328 + 2 * L.g)), dB = prim::h2f(prim::lds_u16(blk + 3328 + 2 * (L.g + 8)));
#pragma unroll
        for (int v = 0; v < NV; v++) {
            accA[v] = prim::fma(dA, combine(PA0[v], PA1[v], L), accA[v]);
            accB[v] = prim::fma(dB, combine(PB0[v], PB1[v], L), accB[v]);
        }
    }
};

// ---- Q8_0: a block is 4 GGUF blocks (128 values) ---------------------------------------------
struct Q80 {
    static constexpr int FMT = 8;
    static constexpr int STEP_BYTES = 2176;
    static constexpr int STEP = 128;
    static constexpr int SV_GRAN = 0;
    static constexpr float PRESCALE = 1.0f;
    SLAI_HD static uint32_t boff(int t) { return 32 * (t >> 1) + 16 * (t & 1); }
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const uint32_t ba = L.bbase + (uint32_t)step * L.bmul;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const int b = 2 * ci + (L.t >> 1);  // GGUF block inside the step
            const uint4 qA = prim::lds16(blk + 128 + (ci * 2) * 512 + 16 * L.lane), qB = prim::lds16(blk + 128 + (ci * 2 + 1) * 512 + 16 * L.lane);
            const uint4 bv = prim::lds16(ba + 64 * ci);
            int c[4];
            prim::mma_i8<false, true>(c, qA.x, qB.x, qA.y, qB.y, bv.x, bv.y);
            prim::mma_i8<false, false>(c, qA.z, qB.z, qA.w, qB.w, bv.z, bv.w);
            const float sA = prim::h2f(prim::lds_u16(blk + 8 * L.g + 2 * b)), sB = prim::h2f(prim::lds_u16(blk + 8 * (L.g + 8) + 2 * b));
            accA = prim::fma(sA, combine(c[0], c[1], L), accA);
            accB = prim::fma(sB, combine(c[2], c[3], L), accB);
        }
    }
    template <int NV>
    SLAI_HD static void compute_batch(uint32_t blk, int step, const LaneCtx& L, const Smem& S, uint32_t bvs, uint32_t svs, float (&accA)[NV],
                                      float (&accB)[NV]) {
        (void)S; (void)svs;
        const uint32_t ba = L.bbase + (uint32_t)step * L.bmul;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const int b = 2 * ci + (L.t >> 1);
            const uint4 qA = prim::lds16(blk + 128 + (ci * 2) * 512 + 16 * L.lane), qB = prim::lds16(blk + 128 + (ci * 2 + 1) * 512 + 16 * L.lane);
            const float sA = prim::h2f(prim::lds_u16(blk + 8 * L.g + 2 * b)), sB = prim::h2f(prim::lds_u16(blk + 8 * (L.g + 8) + 2 * b));
#pragma unroll
            for (int v = 0; v < NV; v++) {
                const uint4 bv = prim::lds16(ba + (uint32_t)v * bvs + 64 * ci);
                int c[4];
                prim::mma_i8<false, true>(c, qA.x, qB.x, qA.y, qB.y, bv.x, bv.y);
                prim::mma_i8<false, false>(c, qA.z, qB.z, qA.w, qB.w, bv.z, bv.w);
                accA[v] = prim::fma(sA, combine(c[0], c[1], L), accA[v]);
                accB[v] = prim::fma(sB, combine(c[2], c[3], L), accB[v]);
            }
        }
    }
};

}  // namespace gemvfmt
