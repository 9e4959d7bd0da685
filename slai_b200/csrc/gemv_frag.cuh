// Per-lane building blocks of the dequant-GEMV kernels: turning packed GGUF quants into the f16
// A-fragments of mma.sync.m16n8k16, and the matching layout of the activation vector.
//
// How a quantised GEMV is mapped onto the tensor cores without changing its result:
//   * A warp owns a tile of 16 matrix rows.  Lane (g = lane/4, t = lane%4) feeds rows g and g+8, and
//     of every 64-byte run of packed quants of those rows it loads the 16-byte chunk number t.
//   * The integer quants are exact in f16, so `sum_k q_k * v_k` is computed by the MMA with f32
//     accumulation; the block scales (d*sc, dmin*m, ...) are applied in f32 afterwards.
//   * The f32 activation v_k is split into two f16 numbers hi+lo (after a power-of-two scaling of the
//     whole vector), which occupy two of the eight MMA columns, so the product keeps ~22 bits.
//   * The remaining columns separate the sub-blocks that have different scales: B holds the activations
//     of sub-block p only in column pair p, so accumulator column pair p is the sum for sub-block p.
//   * Within every group of four consecutive k the activation halves are stored in the order
//     [0,2,1,3], which is the order in which the nibble tricks below produce f16 pairs.
//
// Everything here is __host__ __device__ so that the index arithmetic is unit-tested on the CPU with an
// emulated MMA (tests/host_emul.cpp).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#define SLAI_HD __host__ __device__ __forceinline__

namespace frag {

SLAI_HD uint32_t h2_sub(uint32_t a, uint32_t b) {
#ifdef __CUDA_ARCH__
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
#else
    __half2 x, y;
    memcpy(&x, &a, 4);
    memcpy(&y, &b, 4);
    __half2 r = __floats2half2_rn(__low2float(x) - __low2float(y), __high2float(x) - __high2float(y));
    uint32_t d;
    memcpy(&d, &r, 4);
    return d;
#endif
}
SLAI_HD uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
#ifdef __CUDA_ARCH__
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
#else
    __half2 x, y, z;
    memcpy(&x, &a, 4);
    memcpy(&y, &b, 4);
    memcpy(&z, &c, 4);
    __half2 r = __floats2half2_rn(__low2float(x) * __low2float(y) + __low2float(z),
                                  __high2float(x) * __high2float(y) + __high2float(z));
    uint32_t d;
    memcpy(&d, &r, 4);
    return d;
#endif
}

// f16x2 constants
constexpr uint32_t H2_1024 = 0x64006400u;   // (1024, 1024): mantissa ulp is 1 in [1024, 2048)
constexpr uint32_t H2_1056 = 0x64206420u;   // 1024 + 32
constexpr uint32_t H2_1152 = 0x64806480u;   // 1024 + 128
constexpr uint32_t H2_1_16 = 0x2C002C00u;   // 1/16
constexpr uint32_t H2_M64 = 0xD400D400u;    // -64
constexpr uint32_t H2_M96 = 0xD600D600u;    // -96

// Position of element k inside its group of four in the staged activation arrays.
SLAI_HD int perm4(int k) { return (k & ~3) | ((k & 1) << 1) | ((k >> 1) & 1); }

// ---- 4-bit (Q4_K) -----------------------------------------------------------------------------
// Word x holds 4 bytes = 4 low nibbles (sub-block A) and 4 high nibbles (sub-block B).
// sel = 0 -> bytes 0 and 2, sel = 1 -> bytes 1 and 3.  Results are exact f16 pairs of the nibbles.
SLAI_HD void q4_pair(uint32_t x, int sel, uint32_t& lo, uint32_t& hi) {
    const uint32_t xs = sel ? (x >> 8) : x;
    lo = h2_sub((xs & 0x000F000Fu) | H2_1024, H2_1024);
    hi = h2_fma((xs & 0x00F000F0u) | H2_1024, H2_1_16, H2_M64);
}

// ---- 5-bit (Q5_K) -----------------------------------------------------------------------------
// hw = (qh word) >> (2*G): per byte, bit 0 is the fifth bit of the low-nibble element and bit 1 the
// fifth bit of the high-nibble element.
SLAI_HD void q5_pair(uint32_t x, uint32_t hw, int sel, uint32_t& lo, uint32_t& hi) {
    const uint32_t xs = sel ? (x >> 8) : x;
    const uint32_t hs = sel ? (hw >> 8) : hw;
    lo = h2_sub((xs & 0x000F000Fu) | ((hs & 0x00010001u) << 4) | H2_1024, H2_1024);
    hi = h2_fma((xs & 0x00F000F0u) | ((hs & 0x00020002u) << 7) | H2_1024, H2_1_16, H2_M64);
}

// ---- 6-bit (Q6_K) -----------------------------------------------------------------------------
// x: word of ql; hw = (qh word) >> (2*(c/2)) where c is the 16-byte chunk of the 64-byte ql half:
// per byte, bits 0-1 complete the low nibble, bits 4-5 the high nibble.  Results are q-32.
SLAI_HD void q6_pair(uint32_t x, uint32_t hw, int sel, uint32_t& lo, uint32_t& hi) {
    const uint32_t xs = sel ? (x >> 8) : x;
    const uint32_t hs = sel ? (hw >> 8) : hw;
    lo = h2_sub((xs & 0x000F000Fu) | ((hs & 0x00030003u) << 4) | H2_1024, H2_1056);
    hi = h2_fma((xs & 0x00F000F0u) | ((hs & 0x00300030u) << 4) | H2_1024, H2_1_16, H2_M96);
}

// ---- 8-bit (Q8_0) -----------------------------------------------------------------------------
// x: four int8.  e = bytes (0,2), o = bytes (1,3) as exact f16 pairs.
SLAI_HD uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t s) {
#ifdef __CUDA_ARCH__
    return __byte_perm(a, b, s);
#else
    uint8_t src[8];
    memcpy(src, &a, 4);
    memcpy(src + 4, &b, 4);
    uint32_t r = 0;
    for (int i = 0; i < 4; i++) r |= (uint32_t)src[(s >> (4 * i)) & 7] << (8 * i);
    return r;
#endif
}
SLAI_HD void q8_pair(uint32_t x, uint32_t& e, uint32_t& o) {
    const uint32_t u = x ^ 0x80808080u;  // q + 128 in [0, 255]
    e = h2_sub(byte_perm(u, 0x64646464u, 0x4240), H2_1152);
    o = h2_sub(byte_perm(u, 0x64646464u, 0x4341), H2_1152);
}

// ---- K-quant 6-bit scale / min of sub-block j from the 12 packed bytes (three words s0,s1,s2),
// quantization.rs:381-389.
SLAI_HD void scale_min_k4(int j, uint32_t s0, uint32_t s1, uint32_t s2, uint32_t& sc, uint32_t& m) {
    const int sh = 8 * (j & 3);
    const uint32_t a = (s0 >> sh) & 0xFF, b = (s1 >> sh) & 0xFF, c = (s2 >> sh) & 0xFF;
    if (j < 4) {
        sc = a & 63;
        m = b & 63;
    } else {
        sc = (c & 0xF) | ((a >> 6) << 4);
        m = (c >> 4) | ((b >> 6) << 4);
    }
}

// ---- Which staged activations a lane feeds into the B operand --------------------------------
// All offsets are in f16 elements relative to the start of the current K step in the staged hi (or
// lo) array; -1 means "this lane contributes zeros".
struct BSel {
    int off;   // element offset of 16 consecutive staged halves (32 bytes), or -1
    int lo;    // 0: read the hi array, 1: read the lo array
};

// Q4_K / Q5_K, chunk ci (0: sub-blocks 0-3, 1: sub-blocks 4-7), register slot (0: b0, 1: b1).
SLAI_HD BSel bsel_k4(int lane, int ci, int slot) {
    const int g = lane >> 2, t = lane & 3, p = g >> 1;
    BSel r;
    r.lo = g & 1;
    const bool active = ((t >> 1) == (p >> 1)) && ((p & 1) == slot);
    r.off = active ? 32 * (4 * ci + p) + 16 * (t & 1) : -1;
    return r;
}
// Q6_K, half h of the super-block (128 elements), register slot; hi and lo arrays are both read.
SLAI_HD int bsel_q6(int lane, int slot) {
    const int g = lane >> 2, t = lane & 3;
    const bool active = slot == 0 ? (g == t) : (g == 4 + t);
    return active ? 16 * g : -1;
}
// Q8_0, chunk ci of a 128-element step (blocks 2ci, 2ci+1); both b0 and b1 come from the same 32 bytes.
SLAI_HD BSel bsel_q8(int lane, int ci) {
    const int g = lane >> 2, t = lane & 3, p = g >> 1;
    BSel r;
    r.lo = g & 1;
    const bool active = ((p >> 1) == ci) && ((t >> 1) == (p & 1));
    r.off = active ? 32 * p + 16 * (t & 1) : -1;
    return r;
}

}  // namespace frag
