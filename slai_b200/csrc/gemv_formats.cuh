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
// Predicated loads: lanes with pred == false get zeros and do not touch shared memory (no branch).
SLAI_HD uint4 lds16_if(bool pred, uint32_t addr) {
#ifdef __CUDA_ARCH__
    uint4 r;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\tmov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t"
        "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "=&r"(r.x), "=&r"(r.y), "=&r"(r.z), "=&r"(r.w)
        : "r"(addr), "r"((uint32_t)pred));
    return r;
#else
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (pred) memcpy(&r, hostemu::warp->smem + addr, 16);
    return r;
#endif
}
SLAI_HD uint2 lds8_if(bool pred, uint32_t addr) {
#ifdef __CUDA_ARCH__
    uint2 r;
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %3, 0;\n\tmov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\t@p ld.shared.v2.u32 {%0,%1}, [%2];\n\t}"
                 : "=&r"(r.x), "=&r"(r.y)
                 : "r"(addr), "r"((uint32_t)pred));
    return r;
#else
    uint2 r = make_uint2(0u, 0u);
    if (pred) memcpy(&r, hostemu::warp->smem + addr, 8);
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
// D = A(16x32, row, s8) * B(32x8, col, s8) + D (s32).  Lane (g = lane/4, t = lane%4):
//   a0 = A[g][4t..4t+3], a1 = A[g+8][4t..], a2 = A[g][16+4t..], a3 = A[g+8][16+4t..]   (4 x s8 per register)
//   b0 = B[4t..4t+3][g], b1 = B[16+4t..][g];   c0,c1 = D[g][2t..2t+1], c2,c3 = D[g+8][2t..2t+1]
SLAI_HD void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
#ifdef __CUDA_ARCH__
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
#else
    hostemu::Warp* W = hostemu::warp;
    const int lane = hostemu::lane;
    W->a[lane][0] = a0; W->a[lane][1] = a1; W->a[lane][2] = a2; W->a[lane][3] = a3;
    W->b[lane][0] = b0; W->b[lane][1] = b1;
    pthread_barrier_wait(&W->bar);
    auto A = [&](int row, int k) {
        const int l = (row & 7) * 4 + ((k & 15) >> 2);
        const int reg = (row >= 8 ? 1 : 0) + (k >= 16 ? 2 : 0);
        return (int)(signed char)((W->a[l][reg] >> (8 * (k & 3))) & 0xFF);
    };
    auto B = [&](int k, int n) {
        const int l = n * 4 + ((k & 15) >> 2);
        const int reg = k >= 16 ? 1 : 0;
        return (int)(signed char)((W->b[l][reg] >> (8 * (k & 3))) & 0xFF);
    };
    const int g = lane >> 2, t = lane & 3;
    for (int i = 0; i < 4; i++) {
        const int row = g + (i >= 2 ? 8 : 0), col = 2 * t + (i & 1);
        int s = c[i];
        for (int k = 0; k < 32; k++) s += A(row, k) * B(k, col);
        c[i] = s;
    }
    pthread_barrier_wait(&W->bar);
#endif
}

}  // namespace prim

namespace gemvfmt {

using namespace frag;

// Shared-space byte addresses of the staged activation vector: four planes of s8 digits (plane p at
// dig + p*plane, element k at byte k) and per-sub-block digit sums (4 x s32 per sub-block of SV_GRAN elements).
struct Smem {
    uint32_t dig, plane, sv;
};

struct LaneCtx {
    int lane, g, t;
    bool bact;        // this lane supplies non-zero B values (its column belongs to its own sub-block)
    uint32_t bdig;    // digit plane of this lane's B column (g & 3)
    float wd0, wd1;   // weights of the two digits whose sums this lane holds (digits 2(t&1), 2(t&1)+1)
};

SLAI_HD void lane_init(LaneCtx& L, int lane, const Smem& S) {
    L.lane = lane;
    L.g = lane >> 2;
    L.t = lane & 3;
    L.bact = (L.t >> 1) == (L.g >> 2);
    L.bdig = S.dig + (L.g & 3) * S.plane;
    L.wd0 = digit_weight(2 * (L.t & 1));
    L.wd1 = digit_weight(2 * (L.t & 1) + 1);
}

SLAI_HD float combine(int p0, int p1, const LaneCtx& L) { return prim::fma((float)p1, L.wd1, (float)p0 * L.wd0); }

// Every format provides
//   STEP      elements of K per tile-step block          SV_GRAN  elements per digit-sum entry (0: none)
//   compute   one tile-step block at shared address `blk` (K step number `step`): accumulates rows g and g+8
// ---- Q4_K / Q5_K ---------------------------------------------------------------------------
template <bool FIVE>
struct K45 {
    static constexpr int FMT = FIVE ? 13 : 12;
    static constexpr int STEP = 256;
    static constexpr int SV_GRAN = 32;
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const uint4 hA = prim::lds16(blk + 16 * L.g), hB = prim::lds16(blk + 16 * (L.g + 8));
        uint4 hqA = hA, hqB = hB;
        if (FIVE) {
            hqA = prim::lds16(blk + 256 + 32 * L.g + 16 * (L.t & 1));
            hqB = prim::lds16(blk + 256 + 32 * (L.g + 8) + 16 * (L.t & 1));
        }
        const uint32_t q0 = blk + (FIVE ? 768 : 256) + 16 * L.lane;
        const int tsh = 16 * (L.t >> 1);  // this lane's sub-blocks are 2(t>>1)+nib (+4 for ci = 1)
        const uint32_t yA = hA.y >> tsh, zA = hA.z >> tsh, wA = hA.w >> tsh;
        const uint32_t yB = hB.y >> tsh, zB = hB.z >> tsh, wB = hB.w >> tsh;
        int PA0 = 0, PA1 = 0, QA0 = 0, QA1 = 0, PB0 = 0, PB1 = 0, QB0 = 0, QB1 = 0;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint4 qA = prim::lds16(q0 + (ci * 2) * 512), qB = prim::lds16(q0 + (ci * 2 + 1) * 512);
            const int hsh = 2 * ((L.t >> 1) + 2 * ci);  // Q5_K: 2 * (64-element group index)
            const uint32_t hAx = hqA.x >> hsh, hAy = hqA.y >> hsh, hAz = hqA.z >> hsh, hAw = hqA.w >> hsh;
            const uint32_t hBx = hqB.x >> hsh, hBy = hqB.y >> hsh, hBz = hqB.z >> hsh, hBw = hqB.w >> hsh;
#pragma unroll
            for (int nib = 0; nib < 2; nib++) {
                const int j = 4 * ci + 2 * (L.t >> 1) + nib;  // sub-block (of 32) inside the super-block
                const uint4 bv = prim::lds16_if(L.bact, L.bdig + 256 * step + 32 * j + 16 * (L.t & 1));
                int c[4] = {0, 0, 0, 0};
                if (FIVE) {
                    prim::mma_s8(c, q5_nibs(qA.x, hAx, nib), q5_nibs(qB.x, hBx, nib), q5_nibs(qA.y, hAy, nib), q5_nibs(qB.y, hBy, nib), bv.x, bv.y);
                    prim::mma_s8(c, q5_nibs(qA.z, hAz, nib), q5_nibs(qB.z, hBz, nib), q5_nibs(qA.w, hAw, nib), q5_nibs(qB.w, hBw, nib), bv.z, bv.w);
                } else {
                    prim::mma_s8(c, q4_nibs(qA.x, nib), q4_nibs(qB.x, nib), q4_nibs(qA.y, nib), q4_nibs(qB.y, nib), bv.x, bv.y);
                    prim::mma_s8(c, q4_nibs(qA.z, nib), q4_nibs(qB.z, nib), q4_nibs(qA.w, nib), q4_nibs(qB.w, nib), bv.z, bv.w);
                }
                const uint2 sv = prim::lds8(S.sv + 16 * (step * 8 + j) + 8 * (L.t & 1));
                int scA, mA, scB, mB;
                if (ci == 0) {
                    scA = (yA >> (8 * nib)) & 63; mA = (zA >> (8 * nib)) & 63;
                    scB = (yB >> (8 * nib)) & 63; mB = (zB >> (8 * nib)) & 63;
                } else {
                    scA = ((wA >> (8 * nib)) & 0xF) | (((yA >> (8 * nib + 6)) & 3) << 4);
                    mA = ((wA >> (8 * nib + 4)) & 0xF) | (((zA >> (8 * nib + 6)) & 3) << 4);
                    scB = ((wB >> (8 * nib)) & 0xF) | (((yB >> (8 * nib + 6)) & 3) << 4);
                    mB = ((wB >> (8 * nib + 4)) & 0xF) | (((zB >> (8 * nib + 6)) & 3) << 4);
                }
                PA0 += scA * c[0]; PA1 += scA * c[1]; QA0 += mA * (int)sv.x; QA1 += mA * (int)sv.y;
                PB0 += scB * c[2]; PB1 += scB * c[3]; QB0 += mB * (int)sv.x; QB1 += mB * (int)sv.y;
            }
        }
        const float dA = prim::h2f(hA.x & 0xFFFF), mnA = prim::h2f(hA.x >> 16);
        const float dB = prim::h2f(hB.x & 0xFFFF), mnB = prim::h2f(hB.x >> 16);
        accA = prim::fma(dA, combine(PA0, PA1, L), accA);
        accA = prim::fma(-mnA, combine(QA0, QA1, L), accA);
        accB = prim::fma(dB, combine(PB0, PB1, L), accB);
        accB = prim::fma(-mnB, combine(QB0, QB1, L), accB);
    }
};
using Q4K = K45<false>;
using Q5K = K45<true>;

// ---- Q6_K ----------------------------------------------------------------------------------
struct Q6K {
    static constexpr int FMT = 14;
    static constexpr int STEP = 256;
    static constexpr int SV_GRAN = 16;
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        int PA0 = 0, PA1 = 0, PB0 = 0, PB1 = 0;
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
                    const uint2 bv = prim::lds8_if(L.bact, L.bdig + 16 * j + 8 * (L.t & 1));
                    int c[4] = {0, 0, 0, 0};
                    prim::mma_s8(c, q6_nibs(qlA.x, qhA.x >> sh, nib), q6_nibs(qlB.x, qhB.x >> sh, nib), q6_nibs(qlA.y, qhA.y >> sh, nib),
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
};

// ---- Q8_0: a block is 4 GGUF blocks (128 values) ---------------------------------------------
struct Q80 {
    static constexpr int FMT = 8;
    static constexpr int STEP = 128;
    static constexpr int SV_GRAN = 0;
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const int b = 2 * ci + (L.t >> 1);  // GGUF block inside the step
            const uint4 qA = prim::lds16(blk + 128 + (ci * 2) * 512 + 16 * L.lane), qB = prim::lds16(blk + 128 + (ci * 2 + 1) * 512 + 16 * L.lane);
            const uint4 bv = prim::lds16_if(L.bact, L.bdig + 128 * step + 32 * b + 16 * (L.t & 1));
            int c[4] = {0, 0, 0, 0};
            prim::mma_s8(c, qA.x, qB.x, qA.y, qB.y, bv.x, bv.y);
            prim::mma_s8(c, qA.z, qB.z, qA.w, qB.w, bv.z, bv.w);
            const float sA = prim::h2f(prim::lds_u16(blk + 8 * L.g + 2 * b)), sB = prim::h2f(prim::lds_u16(blk + 8 * (L.g + 8) + 2 * b));
            accA = prim::fma(sA, combine(c[0], c[1], L), accA);
            accB = prim::fma(sB, combine(c[2], c[3], L), accB);
        }
    }
};

}  // namespace gemvfmt
