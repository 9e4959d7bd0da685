// Per-format MMA bodies of the dequant-GEMV kernel (see gemv.cu for the kernel shape, layout.cuh for the
// tile-step blocks they read from shared memory and gemv_frag.cuh for the fragment mapping).  The functions
// are written against a small set of primitives (shared loads, the m16n8k16 MMA) that have a device
// implementation in PTX
// and a host implementation in which 32 CPU threads play the lanes of a warp, so the very same source is
// exercised by the CPU test-suite (tests/host_emul.cpp) before it ever runs on a GPU.
#pragma once
#include "gemv_frag.cuh"

#ifndef __CUDA_ARCH__
#include <pthread.h>
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

SLAI_HD uint4 ldg16(const void* p) {
#ifdef __CUDA_ARCH__
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
#else
    uint4 r;
    memcpy(&r, p, 16);
    return r;
#endif
}
SLAI_HD uint32_t ldg2(const void* p) {
#ifdef __CUDA_ARCH__
    unsigned short r;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
#else
    unsigned short r;
    memcpy(&r, p, 2);
    return r;
#endif
}
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
SLAI_HD float lds_f32(uint32_t addr) {
#ifdef __CUDA_ARCH__
    float r;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(r) : "r"(addr));
    return r;
#else
    float r;
    memcpy(&r, hostemu::warp->smem + addr, 4);
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
// D = A(16x16, row) * B(16x8, col) + D, f16 inputs, f32 accumulation.  Lane (g = lane/4, t = lane%4):
//   a0 = A[g][2t..2t+1], a1 = A[g+8][2t..], a2 = A[g][2t+8..], a3 = A[g+8][2t+8..]
//   b0 = B[2t..2t+1][g], b1 = B[2t+8..2t+9][g];  c0,c1 = D[g][2t..2t+1], c2,c3 = D[g+8][2t..2t+1]
SLAI_HD void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
#ifdef __CUDA_ARCH__
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
#else
    hostemu::Warp* W = hostemu::warp;
    const int lane = hostemu::lane;
    W->a[lane][0] = a0; W->a[lane][1] = a1; W->a[lane][2] = a2; W->a[lane][3] = a3;
    W->b[lane][0] = b0; W->b[lane][1] = b1;
    pthread_barrier_wait(&W->bar);
    auto A = [&](int row, int k) {
        const int l = (row & 7) * 4 + ((k & 7) >> 1);
        const int reg = (row >= 8 ? 1 : 0) + (k >= 8 ? 2 : 0);
        return h2f((W->a[l][reg] >> (16 * (k & 1))) & 0xFFFF);
    };
    auto B = [&](int k, int n) {
        const int l = n * 4 + ((k & 7) >> 1);
        const int reg = k >= 8 ? 1 : 0;
        return h2f((W->b[l][reg] >> (16 * (k & 1))) & 0xFFFF);
    };
    const int g = lane >> 2, t = lane & 3;
    for (int i = 0; i < 4; i++) {
        const int row = g + (i >= 2 ? 8 : 0), col = 2 * t + (i & 1);
        double s = c[i];
        for (int k = 0; k < 16; k++) s += (double)A(row, k) * (double)B(k, col);
        c[i] = (float)s;
    }
    pthread_barrier_wait(&W->bar);
#endif
}

}  // namespace prim

namespace gemvfmt {

using namespace frag;

SLAI_HD uint32_t w4(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Shared-space byte addresses of the staged activation vector: f16 hi / lo arrays in [0,2,1,3] order, 32
// bytes of zeros, and per-32-element sums of the scaled activations.
struct Smem {
    uint32_t hi, lo, zero, sv;
};

struct LaneCtx {
    int lane, g, t;
    // B-operand source addresses (shared space, bytes) and their per-step strides
    uint32_t bp[4];
    uint32_t bs[4];
};

// Every format provides
//   STEP      elements of K per tile-step block
//   init      the lane's B-operand sources
//   compute   one tile-step block at shared address `blk` (K step number `step`): accumulates rows g and g+8
// ---- Q4_K ----------------------------------------------------------------------------------
struct Q4K {
    static constexpr int FMT = 12;
    static constexpr int STEP = 256;
    static constexpr int QOFF = 256;  // start of the lane-ordered quant regions
    static constexpr bool NEED_SV = true;
    SLAI_HD static void init(LaneCtx& L, const Smem& S) {
        for (int ci = 0; ci < 2; ci++)
            for (int slot = 0; slot < 2; slot++) {
                const BSel b = bsel_k4(L.lane, ci, slot);
                const int i = ci * 2 + slot;
                L.bp[i] = b.off < 0 ? S.zero : (b.lo ? S.lo : S.hi) + 2 * b.off;
                L.bs[i] = b.off < 0 ? 0 : 2 * STEP;
            }
    }
    template <bool FIVE>
    SLAI_HD static void compute_k(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const uint4 hA = prim::lds16(blk + 16 * L.g), hB = prim::lds16(blk + 16 * (L.g + 8));
        const float dA = prim::h2f(hA.x & 0xFFFF), mnA = prim::h2f(hA.x >> 16);
        const float dB = prim::h2f(hB.x & 0xFFFF), mnB = prim::h2f(hB.x >> 16);
        uint4 hqA = hA, hqB = hB;
        if (FIVE) {
            hqA = prim::lds16(blk + 256 + 32 * L.g + 16 * (L.t & 1));
            hqB = prim::lds16(blk + 256 + 32 * (L.g + 8) + 16 * (L.t & 1));
        }
        const uint32_t q0 = blk + (FIVE ? 768 : 256) + 16 * L.lane;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint4 qA = prim::lds16(q0 + (ci * 2) * 512), qB = prim::lds16(q0 + (ci * 2 + 1) * 512);
            const uint32_t p0 = L.bp[ci * 2] + step * L.bs[ci * 2], p1 = L.bp[ci * 2 + 1] + step * L.bs[ci * 2 + 1];
            const uint4 b0a = prim::lds16(p0), b0b = prim::lds16(p0 + 16), b1a = prim::lds16(p1), b1b = prim::lds16(p1 + 16);
            const int sh = 2 * ((L.t >> 1) + 2 * ci);  // Q5_K: 2 * (64-element group index)
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const uint32_t hwA = FIVE ? (w4(hqA, w) >> sh) : 0u, hwB = FIVE ? (w4(hqB, w) >> sh) : 0u;
#pragma unroll
                for (int sel = 0; sel < 2; sel++) {
                    uint32_t a0, a1, a2, a3;
                    if (FIVE) {
                        q5_pair(w4(qA, w), hwA, sel, a0, a2);
                        q5_pair(w4(qB, w), hwB, sel, a1, a3);
                    } else {
                        q4_pair(w4(qA, w), sel, a0, a2);
                        q4_pair(w4(qB, w), sel, a1, a3);
                    }
                    const int i = 2 * w + sel;
                    prim::mma16816(c, a0, a1, a2, a3, i < 4 ? w4(b0a, i) : w4(b0b, i - 4), i < 4 ? w4(b1a, i) : w4(b1b, i - 4));
                }
            }
            const int j = 4 * ci + L.t;
            const float sv = prim::lds_f32(S.sv + 4 * (step * 8 + j));
            uint32_t sc, m;
            scale_min_k4(j, hA.y, hA.z, hA.w, sc, m);
            accA = prim::fma(dA * (float)sc, c[0] + c[1], accA);
            accA = prim::fma(-(mnA * (float)m), sv, accA);
            scale_min_k4(j, hB.y, hB.z, hB.w, sc, m);
            accB = prim::fma(dB * (float)sc, c[2] + c[3], accB);
            accB = prim::fma(-(mnB * (float)m), sv, accB);
        }
    }
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        compute_k<false>(blk, step, L, S, accA, accB);
    }
};

// ---- Q5_K ----------------------------------------------------------------------------------
struct Q5K {
    static constexpr int FMT = 13;
    static constexpr int STEP = 256;
    static constexpr bool NEED_SV = true;
    SLAI_HD static void init(LaneCtx& L, const Smem& S) { Q4K::init(L, S); }
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        Q4K::compute_k<true>(blk, step, L, S, accA, accB);
    }
};

// ---- Q6_K: two halves of 128 elements per block ----------------------------------------------
struct Q6K {
    static constexpr int FMT = 14;
    static constexpr int STEP = 256;
    static constexpr bool NEED_SV = false;
    SLAI_HD static void init(LaneCtx& L, const Smem& S) {
        for (int slot = 0; slot < 2; slot++) {
            const int off = bsel_q6(L.lane, slot);
            L.bp[slot * 2 + 0] = off < 0 ? S.zero : S.hi + 2 * off;
            L.bp[slot * 2 + 1] = off < 0 ? S.zero : S.lo + 2 * off;
            L.bs[slot * 2 + 0] = L.bs[slot * 2 + 1] = off < 0 ? 0 : 2 * 128;  // per half
        }
    }
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const float dA = prim::h2f(prim::lds_u16(blk + 3328 + 2 * L.g)), dB = prim::h2f(prim::lds_u16(blk + 3328 + 2 * (L.g + 8)));
        const int sh = 2 * (L.t >> 1);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int hstep = 2 * step + h;
            const uint4 qlA = prim::lds16(blk + (h * 2) * 512 + 16 * L.lane), qlB = prim::lds16(blk + (h * 2 + 1) * 512 + 16 * L.lane);
            const uint4 qhA = prim::lds16(blk + 2048 + h * 512 + 32 * L.g + 16 * (L.t & 1));
            const uint4 qhB = prim::lds16(blk + 2048 + h * 512 + 32 * (L.g + 8) + 16 * (L.t & 1));
            const uint32_t scA = prim::lds_u16(blk + 3072 + 16 * L.g + 8 * h + 2 * L.t);
            const uint32_t scB = prim::lds_u16(blk + 3072 + 16 * (L.g + 8) + 8 * h + 2 * L.t);
            const uint32_t p0h = L.bp[0] + hstep * L.bs[0], p0l = L.bp[1] + hstep * L.bs[1];
            const uint32_t p1h = L.bp[2] + hstep * L.bs[2], p1l = L.bp[3] + hstep * L.bs[3];
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {  // two groups of 4 MMAs: words 0-1, words 2-3
                const uint4 b0h = prim::lds16(p0h + 16 * hf), b0l = prim::lds16(p0l + 16 * hf);
                const uint4 b1h = prim::lds16(p1h + 16 * hf), b1l = prim::lds16(p1l + 16 * hf);
#pragma unroll
                for (int ww = 0; ww < 2; ww++) {
                    const int w = 2 * hf + ww;
                    const uint32_t hwA = w4(qhA, w) >> sh, hwB = w4(qhB, w) >> sh;
#pragma unroll
                    for (int sel = 0; sel < 2; sel++) {
                        uint32_t a0, a1, a2, a3;
                        q6_pair(w4(qlA, w), hwA, sel, a0, a2);
                        q6_pair(w4(qlB, w), hwB, sel, a1, a3);
                        const int i = 2 * ww + sel;
                        prim::mma16816(c, a0, a1, a2, a3, w4(b0h, i), w4(b1h, i));
                        prim::mma16816(c, a0, a1, a2, a3, w4(b0l, i), w4(b1l, i));
                    }
                }
            }
            // lane holds columns 2t, 2t+1 = sub-blocks 2t, 2t+1 of this half; scales are int8
            const float s0A = (float)(int)(signed char)(scA & 0xFF), s1A = (float)(int)(signed char)(scA >> 8);
            const float s0B = (float)(int)(signed char)(scB & 0xFF), s1B = (float)(int)(signed char)(scB >> 8);
            accA = prim::fma(dA, prim::fma(s0A, c[0], s1A * c[1]), accA);
            accB = prim::fma(dB, prim::fma(s0B, c[2], s1B * c[3]), accB);
        }
    }
};

// ---- Q8_0: a block is 4 GGUF blocks (128 values) ---------------------------------------------
struct Q80 {
    static constexpr int FMT = 8;
    static constexpr int STEP = 128;
    static constexpr bool NEED_SV = false;
    SLAI_HD static void init(LaneCtx& L, const Smem& S) {
        for (int ci = 0; ci < 2; ci++) {
            const BSel b = bsel_q8(L.lane, ci);
            L.bp[ci] = b.off < 0 ? S.zero : (b.lo ? S.lo : S.hi) + 2 * b.off;
            L.bs[ci] = b.off < 0 ? 0 : 2 * STEP;
        }
    }
    SLAI_HD static void compute(uint32_t blk, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const float sA = prim::h2f(prim::lds_u16(blk + 8 * L.g + 2 * L.t)), sB = prim::h2f(prim::lds_u16(blk + 8 * (L.g + 8) + 2 * L.t));
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint4 qA = prim::lds16(blk + 128 + (ci * 2) * 512 + 16 * L.lane), qB = prim::lds16(blk + 128 + (ci * 2 + 1) * 512 + 16 * L.lane);
            const uint32_t p = L.bp[ci] + step * L.bs[ci];
            const uint4 ba = prim::lds16(p), bb = prim::lds16(p + 16);
#pragma unroll
            for (int w = 0; w < 4; w++) {
                uint32_t a0, a1, a2, a3;
                q8_pair(w4(qA, w), a0, a2);
                q8_pair(w4(qB, w), a1, a3);
                prim::mma16816(c, a0, a1, a2, a3, w < 2 ? w4(ba, 2 * w) : w4(bb, 2 * w - 4), w < 2 ? w4(ba, 2 * w + 1) : w4(bb, 2 * w - 3));
            }
        }
        accA = prim::fma(sA, c[0] + c[1], accA);
        accB = prim::fma(sB, c[2] + c[3], accB);
    }
};

}  // namespace gemvfmt
