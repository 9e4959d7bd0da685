// Per-format step loaders and MMA bodies of the dequant-GEMV kernel (see gemv.cu for the kernel shape
// and gemv_frag.cuh for the fragment mapping).  The functions are written against a small set of
// primitives (16-byte global / shared loads, the m16n8k16 MMA) that have a device implementation in PTX
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

// Shared-memory layout (dynamic): [hi: Kp halves][lo: Kp halves][zero: 16 halves][sv: Kp/32 floats]
// [red: WARPS * 32 floats][stat: 64 floats]
struct Smem {
    uint32_t hi, lo, zero, sv;  // shared-space byte addresses
    float* red;
    float* stat;
};

// ---------------------------------------------------------------------------------------------
// Format traits: per-step register payload, loader and MMA body.
// ---------------------------------------------------------------------------------------------
struct LaneCtx {
    int lane, g, t;
    // B-operand source addresses (shared space, bytes) and per-step strides
    uint32_t bp[8];
    uint32_t bs[8];
};

// ---- Q4_K ----------------------------------------------------------------------------------
struct Q4K {
    static constexpr int STEP = 256;
    static constexpr bool NEED_SV = true;
    SLAI_HD static uint32_t aux(int) { return 0u; }
    struct Regs { uint4 hA, hB, qA[2], qB[2]; };
    SLAI_HD static void init(LaneCtx& L, const Smem& S) {
        for (int ci = 0; ci < 2; ci++)
            for (int slot = 0; slot < 2; slot++) {
                const BSel b = bsel_k4(L.lane, ci, slot);
                const int i = ci * 2 + slot;
                L.bp[i] = b.off < 0 ? S.zero : (b.lo ? S.lo : S.hi) + 2 * b.off;
                L.bs[i] = b.off < 0 ? 0 : 2 * STEP;
            }
    }
    SLAI_HD static void load(Regs& r, const uint8_t* rowA, const uint8_t* rowB, int step, const LaneCtx& L) {
        const uint8_t* a = rowA + (size_t)step * 144;
        const uint8_t* b = rowB + (size_t)step * 144;
        r.hA = prim::ldg16(a);
        r.hB = prim::ldg16(b);
        r.qA[0] = prim::ldg16(a + 16 + 16 * L.t);
        r.qB[0] = prim::ldg16(b + 16 + 16 * L.t);
        r.qA[1] = prim::ldg16(a + 80 + 16 * L.t);
        r.qB[1] = prim::ldg16(b + 80 + 16 * L.t);
    }
    SLAI_HD static void compute(const Regs& r, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const float dA = prim::h2f(r.hA.x & 0xFFFF), mnA = prim::h2f(r.hA.x >> 16);
        const float dB = prim::h2f(r.hB.x & 0xFFFF), mnB = prim::h2f(r.hB.x >> 16);
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint32_t p0 = L.bp[ci * 2] + step * L.bs[ci * 2], p1 = L.bp[ci * 2 + 1] + step * L.bs[ci * 2 + 1];
            const uint4 b0a = prim::lds16(p0), b0b = prim::lds16(p0 + 16), b1a = prim::lds16(p1), b1b = prim::lds16(p1 + 16);
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int w = 0; w < 4; w++) {
#pragma unroll
                for (int sel = 0; sel < 2; sel++) {
                    uint32_t a0, a1, a2, a3;
                    q4_pair(w4(r.qA[ci], w), sel, a0, a2);
                    q4_pair(w4(r.qB[ci], w), sel, a1, a3);
                    const int i = 2 * w + sel;
                    prim::mma16816(c, a0, a1, a2, a3, i < 4 ? w4(b0a, i) : w4(b0b, i - 4), i < 4 ? w4(b1a, i) : w4(b1b, i - 4));
                }
            }
            const int j = 4 * ci + L.t;
            const float sv = prim::lds_f32(S.sv + 4 * (step * 8 + j));
            uint32_t sc, m;
            scale_min_k4(j, r.hA.y, r.hA.z, r.hA.w, sc, m);
            accA = prim::fma(dA * (float)sc, c[0] + c[1], accA);
            accA = prim::fma(-(mnA * (float)m), sv, accA);
            scale_min_k4(j, r.hB.y, r.hB.z, r.hB.w, sc, m);
            accB = prim::fma(dB * (float)sc, c[2] + c[3], accB);
            accB = prim::fma(-(mnB * (float)m), sv, accB);
        }
    }
};

// ---- Q5_K ----------------------------------------------------------------------------------
struct Q5K {
    static constexpr int STEP = 256;
    static constexpr bool NEED_SV = true;
    SLAI_HD static uint32_t aux(int) { return 0u; }
    struct Regs { uint4 hA, hB, hqA, hqB, qA[2], qB[2]; };
    SLAI_HD static void init(LaneCtx& L, const Smem& S) { Q4K::init(L, S); }
    SLAI_HD static void load(Regs& r, const uint8_t* rowA, const uint8_t* rowB, int step, const LaneCtx& L) {
        const uint8_t* a = rowA + (size_t)step * 176;
        const uint8_t* b = rowB + (size_t)step * 176;
        r.hA = prim::ldg16(a);
        r.hB = prim::ldg16(b);
        r.hqA = prim::ldg16(a + 16 + 16 * (L.t & 1));
        r.hqB = prim::ldg16(b + 16 + 16 * (L.t & 1));
        r.qA[0] = prim::ldg16(a + 48 + 16 * L.t);
        r.qB[0] = prim::ldg16(b + 48 + 16 * L.t);
        r.qA[1] = prim::ldg16(a + 112 + 16 * L.t);
        r.qB[1] = prim::ldg16(b + 112 + 16 * L.t);
    }
    SLAI_HD static void compute(const Regs& r, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const float dA = prim::h2f(r.hA.x & 0xFFFF), mnA = prim::h2f(r.hA.x >> 16);
        const float dB = prim::h2f(r.hB.x & 0xFFFF), mnB = prim::h2f(r.hB.x >> 16);
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint32_t p0 = L.bp[ci * 2] + step * L.bs[ci * 2], p1 = L.bp[ci * 2 + 1] + step * L.bs[ci * 2 + 1];
            const uint4 b0a = prim::lds16(p0), b0b = prim::lds16(p0 + 16), b1a = prim::lds16(p1), b1b = prim::lds16(p1 + 16);
            const int sh = 2 * ((L.t >> 1) + 2 * ci);  // 2 * (64-element group index)
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const uint32_t hwA = w4(r.hqA, w) >> sh, hwB = w4(r.hqB, w) >> sh;
#pragma unroll
                for (int sel = 0; sel < 2; sel++) {
                    uint32_t a0, a1, a2, a3;
                    q5_pair(w4(r.qA[ci], w), hwA, sel, a0, a2);
                    q5_pair(w4(r.qB[ci], w), hwB, sel, a1, a3);
                    const int i = 2 * w + sel;
                    prim::mma16816(c, a0, a1, a2, a3, i < 4 ? w4(b0a, i) : w4(b0b, i - 4), i < 4 ? w4(b1a, i) : w4(b1b, i - 4));
                }
            }
            const int j = 4 * ci + L.t;
            const float sv = prim::lds_f32(S.sv + 4 * (step * 8 + j));
            uint32_t sc, m;
            scale_min_k4(j, r.hA.y, r.hA.z, r.hA.w, sc, m);
            accA = prim::fma(dA * (float)sc, c[0] + c[1], accA);
            accA = prim::fma(-(mnA * (float)m), sv, accA);
            scale_min_k4(j, r.hB.y, r.hB.z, r.hB.w, sc, m);
            accB = prim::fma(dB * (float)sc, c[2] + c[3], accB);
            accB = prim::fma(-(mnB * (float)m), sv, accB);
        }
    }
};

// ---- Q6_K (row planes: ql | qh | scales | d), one step = half a super-block (128 elements) ---
struct Q6K {
    static constexpr int STEP = 128;
    static constexpr bool NEED_SV = false;
    SLAI_HD static uint32_t aux(int K) { return (uint32_t)(K >> 8); }  // super-blocks per row
    struct Regs { uint4 qlA, qlB, qhA, qhB; uint32_t scA, scB, dA, dB; };
    SLAI_HD static void init(LaneCtx& L, const Smem& S) {
        for (int slot = 0; slot < 2; slot++) {
            const int off = bsel_q6(L.lane, slot);
            L.bp[slot * 2 + 0] = off < 0 ? S.zero : S.hi + 2 * off;
            L.bp[slot * 2 + 1] = off < 0 ? S.zero : S.lo + 2 * off;
            L.bs[slot * 2 + 0] = L.bs[slot * 2 + 1] = off < 0 ? 0 : 2 * STEP;
        }
    }
    // nb = super-blocks per row (plane offsets depend on it); passed through L.bs[7]
    SLAI_HD static void load(Regs& r, const uint8_t* rowA, const uint8_t* rowB, int step, const LaneCtx& L) {
        const int nb = (int)L.bs[7];
        const size_t oql = (size_t)step * 64 + 16 * L.t;                            // 64 ql bytes per half
        const size_t oqh = (size_t)nb * 128 + (size_t)step * 32 + 16 * (L.t & 1);   // 32 qh bytes per half
        const size_t osc = (size_t)nb * 192 + (size_t)step * 8 + 2 * L.t;           // 8 scales per half
        const size_t od = (size_t)nb * 208 + (size_t)(step >> 1) * 2;
        r.qlA = prim::ldg16(rowA + oql);
        r.qlB = prim::ldg16(rowB + oql);
        r.qhA = prim::ldg16(rowA + oqh);
        r.qhB = prim::ldg16(rowB + oqh);
        r.scA = prim::ldg2(rowA + osc);
        r.scB = prim::ldg2(rowB + osc);
        r.dA = prim::ldg2(rowA + od);
        r.dB = prim::ldg2(rowB + od);
    }
    SLAI_HD static void compute(const Regs& r, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        const uint32_t p0h = L.bp[0] + step * L.bs[0], p0l = L.bp[1] + step * L.bs[1];
        const uint32_t p1h = L.bp[2] + step * L.bs[2], p1l = L.bp[3] + step * L.bs[3];
        const int sh = 2 * (L.t >> 1);
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {  // two groups of 4 MMAs: words 0-1, words 2-3
            const uint4 b0h = prim::lds16(p0h + 16 * hf), b0l = prim::lds16(p0l + 16 * hf);
            const uint4 b1h = prim::lds16(p1h + 16 * hf), b1l = prim::lds16(p1l + 16 * hf);
#pragma unroll
            for (int ww = 0; ww < 2; ww++) {
                const int w = 2 * hf + ww;
                const uint32_t hwA = w4(r.qhA, w) >> sh, hwB = w4(r.qhB, w) >> sh;
#pragma unroll
                for (int sel = 0; sel < 2; sel++) {
                    uint32_t a0, a1, a2, a3;
                    q6_pair(w4(r.qlA, w), hwA, sel, a0, a2);
                    q6_pair(w4(r.qlB, w), hwB, sel, a1, a3);
                    const int i = 2 * ww + sel;
                    prim::mma16816(c, a0, a1, a2, a3, w4(b0h, i), w4(b1h, i));
                    prim::mma16816(c, a0, a1, a2, a3, w4(b0l, i), w4(b1l, i));
                }
            }
        }
        // lane holds columns 2t, 2t+1 = sub-blocks 2t, 2t+1 of this half; scales are int8
        const float s0A = (float)(int)(signed char)(r.scA & 0xFF), s1A = (float)(int)(signed char)(r.scA >> 8);
        const float s0B = (float)(int)(signed char)(r.scB & 0xFF), s1B = (float)(int)(signed char)(r.scB >> 8);
        accA = prim::fma(prim::h2f(r.dA), prim::fma(s0A, c[0], s1A * c[1]), accA);
        accB = prim::fma(prim::h2f(r.dB), prim::fma(s0B, c[2], s1B * c[3]), accB);
    }
};

// ---- Q8_0 (row planes: K int8 | K/32 f16 scales), one step = 128 elements (4 blocks) -------
struct Q80 {
    static constexpr int STEP = 128;
    static constexpr bool NEED_SV = false;
    SLAI_HD static uint32_t aux(int K) { return (uint32_t)K; }
    struct Regs { uint4 qA[2], qB[2]; uint32_t sA, sB; };
    SLAI_HD static void init(LaneCtx& L, const Smem& S) {
        for (int ci = 0; ci < 2; ci++) {
            const BSel b = bsel_q8(L.lane, ci);
            L.bp[ci] = b.off < 0 ? S.zero : (b.lo ? S.lo : S.hi) + 2 * b.off;
            L.bs[ci] = b.off < 0 ? 0 : 2 * STEP;
        }
    }
    // K passed through L.bs[7] (offset of the scale plane, and the bound for partial steps)
    SLAI_HD static void load(Regs& r, const uint8_t* rowA, const uint8_t* rowB, int step, const LaneCtx& L) {
        const int K = (int)L.bs[7];
        const int e0 = step * 128 + 16 * L.t, e1 = e0 + 64;
        const uint4 z = make_uint4(0x0, 0x0, 0x0, 0x0);
        r.qA[0] = e0 < K ? prim::ldg16(rowA + e0) : z;
        r.qB[0] = e0 < K ? prim::ldg16(rowB + e0) : z;
        r.qA[1] = e1 < K ? prim::ldg16(rowA + e1) : z;
        r.qB[1] = e1 < K ? prim::ldg16(rowB + e1) : z;
        const int blk = step * 4 + L.t;
        const bool ok = blk * 32 < K;
        r.sA = ok ? prim::ldg2(rowA + K + 2 * blk) : 0;
        r.sB = ok ? prim::ldg2(rowB + K + 2 * blk) : 0;
    }
    SLAI_HD static void compute(const Regs& r, int step, const LaneCtx& L, const Smem& S, float& accA, float& accB) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const uint32_t p = L.bp[ci] + step * L.bs[ci];
            const uint4 ba = prim::lds16(p), bb = prim::lds16(p + 16);
#pragma unroll
            for (int w = 0; w < 4; w++) {
                uint32_t a0, a1, a2, a3;
                q8_pair(w4(r.qA[ci], w), a0, a2);
                q8_pair(w4(r.qB[ci], w), a1, a3);
                prim::mma16816(c, a0, a1, a2, a3, w < 2 ? w4(ba, 2 * w) : w4(bb, 2 * w - 4),
                         w < 2 ? w4(ba, 2 * w + 1) : w4(bb, 2 * w - 3));
            }
        }
        accA = prim::fma(prim::h2f(r.sA), c[0] + c[1], accA);
        accB = prim::fma(prim::h2f(r.sB), c[2] + c[3], accB);
    }
};


}  // namespace gemvfmt
