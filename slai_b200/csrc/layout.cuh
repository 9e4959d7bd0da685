// Device layout of quantized matrices (see common.cuh) and the per-block repacking from GGUF order.
#pragma once
#include <stdint.h>
#include <string.h>
#include "gemv_frag.cuh"

namespace layout {

SLAI_HD int64_t round16(int64_t x) { return (x + 15) & ~(int64_t)15; }

// Bytes between consecutive rows of the device layout.
SLAI_HD int64_t row_stride(int fmt, int64_t K) {
    switch (fmt) {
        case 0: return K * 4;                         // F32
        case 8: return round16(K + K / 16);           // Q8_0: K int8 + K/32 f16
        case 12: return K / 256 * 144;                // Q4_K (file layout)
        case 13: return K / 256 * 176;                // Q5_K (file layout)
        case 14: return round16(K / 256 * 210);       // Q6_K planes
    }
    return 0;
}

// Copy GGUF block number `blk` of a row (raw bytes at `src`) to its place in the device row `dst`.
SLAI_HD void repack_block(int fmt, const uint8_t* src, uint8_t* dst, int64_t blk, int64_t K) {
    if (fmt == 8) {  // [f16 scale][32 x int8]  ->  quant plane, scale plane
        for (int i = 0; i < 32; i++) dst[blk * 32 + i] = src[2 + i];
        dst[K + 2 * blk] = src[0];
        dst[K + 2 * blk + 1] = src[1];
    } else if (fmt == 14) {  // [ql 128][qh 64][scales 16][d 2]  ->  four planes
        const int64_t nb = K / 256;
        for (int i = 0; i < 128; i++) dst[blk * 128 + i] = src[i];
        for (int i = 0; i < 64; i++) dst[nb * 128 + blk * 64 + i] = src[128 + i];
        for (int i = 0; i < 16; i++) dst[nb * 192 + blk * 16 + i] = src[192 + i];
        dst[nb * 208 + blk * 2] = src[208];
        dst[nb * 208 + blk * 2 + 1] = src[209];
    } else {
        const int bb = fmt == 12 ? 144 : fmt == 13 ? 176 : 4;
        for (int i = 0; i < bb; i++) dst[blk * bb + i] = src[i];
    }
}

}  // namespace layout
