// Per-lane building blocks of the dequant-GEMV kernels.
//
// How a quantised GEMV is mapped onto the tensor cores without changing its result:
//   * A warp owns a tile of 16 matrix rows.  Lane (g = lane/4, t = lane%4) feeds rows g and g+8 of the
//     integer MMA m16n8k32 (s8 x s8 -> s32): its A registers are packed quants, four per register, obtained
//     from the GGUF nibbles / bytes with one or two logic instructions (no int->float conversion).
//   * The f32 activation vector is scaled by a power of two and rounded to a 27-bit fixed-point integer
//     V_k, which is split into four signed base-256 digits (V = d3*2^24 + d2*2^16 + d1*2^8 + d0, the low three
//     in [-128, 127]).  The digits occupy four of the eight MMA columns, so `sum_k q_k * V_k` is evaluated
//     exactly in integer arithmetic (the only rounding is that of V_k, relative 2^-26 of max|v|).
//   * The other factor of two in the columns separates two sub-blocks with different scales: lanes t < 2
//     carry one sub-block, lanes t >= 2 another, and B holds the digits of a sub-block only in its own four
//     columns.  Lane t therefore ends up with the sums of *its own* sub-block for digits 2(t&1), 2(t&1)+1.
//   * Block scales are applied in integer (6-bit / 8-bit scale x s32 sum) and converted to f32 once per
//     super-block, then multiplied by the f16 super-block scale.
//
// Everything here is __host__ __device__ so that the index arithmetic is unit-tested on the CPU with an
// emulated MMA (tests/host_emul.cpp).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#define SLAI_HD __host__ __device__ __forceinline__

namespace frag {

constexpr uint32_t M4 = 0x0F0F0F0Fu;

// ---- A operands: four quants per register -------------------------------------------------------
// Q4_K: low or high nibbles of a qs word.
SLAI_HD uint32_t q4_nibs(uint32_t x, int nib) { return nib ? ((x >> 4) & M4) : (x & M4); }
// Q5_K: hw = (qh word) >> (2*G): per byte, bit 0 completes the low nibble, bit 1 the high nibble.
SLAI_HD uint32_t q5_nibs(uint32_t x, uint32_t hw, int nib) {
    return nib ? (((x >> 4) & M4) | ((hw & 0x02020202u) << 3)) : ((x & M4) | ((hw & 0x01010101u) << 4));
}
// Q6_K: hs = (qh word) >> (2*pair + 4*nib): per byte, bits 0-1 are the upper two bits.  Result is q (0..63);
// the -32 offset is applied to the integer sums.
SLAI_HD uint32_t q6_nibs(uint32_t x, uint32_t hs, int nib) {
    return (nib ? ((x >> 4) & M4) : (x & M4)) | ((hs & 0x03030303u) << 4);
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

// ---- activation digits -------------------------------------------------------------------------
// V (|V| <= 2^26 + 1) -> four signed base-256 digits, V = d3*2^24 + d2*2^16 + d1*2^8 + d0 with d0..d2 in [-128, 127]:
// adding 0x808080 turns the three low bytes of the two's-complement word into the digits biased by 128, and flipping
// their top bits removes the bias -- two instructions for all four digits, packed one per byte (byte i = digit i).
SLAI_HD uint32_t digits_word(int V) { return ((uint32_t)V + 0x00808080u) ^ 0x00808080u; }
// Transpose four elements' digit words into four plane words (plane p = digit p of the four elements, in order).
SLAI_HD uint32_t perm_bytes(uint32_t a, uint32_t b, uint32_t sel) {
#ifdef __CUDA_ARCH__
    return __byte_perm(a, b, sel);
#else
    const uint64_t both = ((uint64_t)b << 32) | a;
    uint32_t r = 0;
    for (int i = 0; i < 4; i++) r |= (uint32_t)((both >> (8 * ((sel >> (4 * i)) & 7))) & 0xFF) << (8 * i);
    return r;
#endif
}
SLAI_HD void digit_planes(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t (&plane)[4]) {
    const uint32_t t0 = perm_bytes(w0, w1, 0x5140), t1 = perm_bytes(w2, w3, 0x5140);
    const uint32_t t2 = perm_bytes(w0, w1, 0x7362), t3 = perm_bytes(w2, w3, 0x7362);
    plane[0] = perm_bytes(t0, t1, 0x5410);
    plane[1] = perm_bytes(t0, t1, 0x7632);
    plane[2] = perm_bytes(t2, t3, 0x5410);
    plane[3] = perm_bytes(t2, t3, 0x7632);
}
// weight of digit plane i: 256^i
SLAI_HD float digit_weight(int i) { return i == 0 ? 1.0f : i == 1 ? 256.0f : i == 2 ? 65536.0f : 16777216.0f; }

}  // namespace frag
