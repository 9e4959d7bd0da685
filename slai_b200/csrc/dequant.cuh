// One dequantised element read from the tile-major device layout (layout.cuh), with the reference's rounding
// sequence.  Shared by the bit-exact dump / embedding lookup (ops.cu) and the prompt GEMM's operand staging
// (prefill.cu).
#pragma once
#include "common.cuh"
#include "gemv_frag.cuh"
#include "layout.cuh"

__device__ __forceinline__ float dev_h2f(unsigned int bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// One dequantised element, read from the tile-major layout, with the reference's rounding sequence (no FMA
// contraction):
//   Q8_0: q * scale                         quantization.rs:38-41
//   Q4_K/Q5_K: (d*sc)*q - (dmin*m)          quantization.rs:357-371, 288-307
//   Q6_K: (d*scale)*q                       quantization.rs:233-236
__device__ __forceinline__ float dequant_elem(int fmt, const uint8_t* data, long long K, long long row, long long k) {
    const long long ns = layout::num_steps(fmt, K);
    const int r = (int)(row & 15);
    if (fmt == SLAI_FMT_Q8_0) {
        const uint8_t* b = data + ((row >> 4) * ns + (k >> 7)) * 2176;
        const int e = (int)(k & 127);
        const int q = (int)(signed char)b[layout::qbyte_off(128, r, e)];
        const unsigned int sb = b[8 * r + 2 * (e >> 5)] | (b[8 * r + 2 * (e >> 5) + 1] << 8);
        return __fmul_rn((float)q, dev_h2f(sb));
    }
    const uint8_t* b = data + ((row >> 4) * ns + (k >> 8)) * layout::step_bytes(fmt);
    const int e = (int)(k & 255);
    if (fmt == SLAI_FMT_Q4_K || fmt == SLAI_FMT_Q5_K) {
        const uint8_t* h = b + layout::K45_HDR_ROW * r;
        const float d = dev_h2f(h[0] | (h[1] << 8)), mn = dev_h2f(h[2] | (h[3] << 8));
        const int G = e >> 6, half = (e >> 5) & 1, l = e & 31;
        const uint8_t qb = b[layout::qbyte_off(fmt == SLAI_FMT_Q4_K ? layout::K45_HDR : layout::K45_HDR + 512, r, 32 * G + l)];
        int q = half ? (qb >> 4) : (qb & 0xF);
        if (fmt == SLAI_FMT_Q5_K) q += ((b[layout::K45_HDR + 32 * r + l] >> (2 * G + half)) & 1) ? 16 : 0;
        const uint32_t sc = h[layout::k45_sc_off(2 * G + half)], m = h[12 + 2 * G + half];  // unpacked at upload
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(mn, (float)m);
        return __fsub_rn(__fmul_rn(d1, (float)q), m1);
    }
    // Q6_K
    const int hf = e >> 7, rr = e & 127, quarter = rr >> 5, l = rr & 31;
    const uint8_t qlb = b[layout::q6_ql_off(r, 64 * hf + l + 32 * (quarter & 1))];
    const int nib = quarter >= 2 ? (qlb >> 4) : (qlb & 0xF);
    const uint8_t qhb = b[layout::q6_qh_off(r, 32 * hf + l)];
    const int q = (nib | (((qhb >> (2 * quarter)) & 3) << 4)) - 32;
    const int sc = (int)(signed char)b[3072 + 16 * r + 8 * hf + (l >> 4) + 2 * quarter];
    const float d = dev_h2f(b[3328 + 2 * r] | (b[3328 + 2 * r + 1] << 8));
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
}

