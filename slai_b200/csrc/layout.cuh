// Device layout of quantized matrices, and the placement of GGUF blocks into it.
//
// A matrix is stored tile-major for streaming: rows are grouped into tiles of 16, the K dimension into
// steps (256 elements; 128 for Q8_0), and the packed data of one (tile, step) is one contiguous,
// 16-byte aligned "tile-step block":
//
//     data = [tile 0][tile 1]...      tile = [step 0][step 1]...      step = SB bytes (below)
//
// so the 16 rows x K-range handled by one warp is a single contiguous byte range that a bulk asynchronous
// copy brings into shared memory, and inside a block the 16-byte chunks are ordered so that the 32 lanes
// of a warp read consecutive chunks (no bank conflicts).  The byte count equals the GGUF file's (plus zero
// padding of the last tile / last Q8_0 step).
//
//   lane = 4*g + t,  g = row & 7,  ab = row >> 3 (rows 0-7 feed MMA rows g, rows 8-15 feed rows g+8)
//
//   Q4_K  (2368 B): [hdr 16 x 20B] [q(ci,ab): 32 lanes x 16B] for ci = 0,1 / ab = 0,1
//                   lane (g,t) of q(ci,ab) holds qs bytes 16*(4ci+t) .. +15 of row g + 8ab
//                   hdr of row r: f16 d, f16 dmin, then the sixteen 6-bit scales / minima of the block unpacked to
//                   one byte each (get_scale_min_k4, quantization.rs:381-389, is applied once at upload instead
//                   of per token): sc of sub-blocks 0,1,4,5 | sc of sub-blocks 2,3,6,7 | m of sub-blocks 0..7.
//                   The unpacking adds 4 bytes per 144-byte GGUF block (2.8 %).
//   Q5_K  (2880 B): [hdr 16 x 20B] [qh 16 x 32B] [q(ci,ab) as Q4_K]
//   Q6_K  (3360 B): [ql(h,pair,ab): 32 lanes x 8B] [qh(h,ab): 32 lanes x 8B] [scales 16 x 16B] [d 16 x 2B]
//                   lane (g,t) of ql(h,pair,ab) holds ql bytes 64h + 16(2 pair + t/2) + 8(t%2) .. +7 and lane
//                   (g,t) of qh(h,ab) holds qh bytes 32h + 8t .. +7 of row g + 8ab: two lanes carry one
//                   16-element sub-block, so an MMA sees two sub-blocks
//   Q8_0  (2176 B): [scales 16 rows x 4 x f16] [q(ci,ab): 32 lanes x 16B]; a step is 4 blocks (128 values),
//                   lane (g,t) of q(ci,ab) holds the int8 values 64ci + 16t .. +15 of the step
//   F32           : dense row-major (no tiling).
#pragma once
#include <stdint.h>
#include <string.h>
#include "gemv_frag.cuh"

namespace layout {

SLAI_HD int step_elems(int fmt) { return fmt == 8 ? 128 : 256; }
SLAI_HD int step_bytes(int fmt) {
    switch (fmt) {
        case 8: return 2176;
        case 12: return 2368;
        case 13: return 2880;
        case 14: return 3360;
    }
    return 0;
}
SLAI_HD int64_t num_steps(int fmt, int64_t K) { return (K + step_elems(fmt) - 1) / step_elems(fmt); }
SLAI_HD int64_t num_tiles(int64_t rows) { return (rows + 15) / 16; }
// Bytes of a matrix with `rows` rows (padded to whole tiles).
SLAI_HD int64_t matrix_bytes(int fmt, int64_t rows, int64_t K) {
    if (fmt == 0) return rows * K * 4;
    return num_tiles(rows) * num_steps(fmt, K) * step_bytes(fmt);
}
SLAI_HD int64_t tile_bytes(int fmt, int64_t K) { return num_steps(fmt, K) * step_bytes(fmt); }

// Q4_K / Q5_K block header: 20 bytes per row (see the table above).  Byte of the scale of sub-block j inside a
// row's header: a lane serves sub-blocks 4 ci + 2 h + nib (h = t >> 1) and finds its four scales in one word.
constexpr int K45_HDR_ROW = 20;
constexpr int K45_HDR = 16 * K45_HDR_ROW;
SLAI_HD int k45_sc_off(int j) {
    const int ci = j >> 2, h = (j >> 1) & 1, nib = j & 1;
    return 4 + 4 * h + 2 * ci + nib;
}

// Offset, inside a tile-step block, of byte `idx` of the packed quant array (qs / ql / int8 values of the
// step) of row r.  The array is cut into 16-byte chunks c = idx/16; chunk c = 4*ci + t goes to lane 4g+t of
// the lane-ordered region (ci, ab).
SLAI_HD int qbyte_off(int region0, int r, int idx) {
    const int c = idx >> 4, ci = c >> 2, t = c & 3, g = r & 7, ab = r >> 3;
    return region0 + (ci * 2 + ab) * 512 + 16 * (4 * g + t) + (idx & 15);
}

// Q6_K: offsets of ql byte idx (0..127) and qh byte idx (0..63) of row r.  The 64 ql bytes of half h are cut
// into 8-byte pieces; piece (chunk c = idx/16 within the half, half-chunk) goes to lane 4g + 2(c&1) + piece of
// region (h, pair = c/2, ab); the 32 qh bytes of half h go, 8 per lane, to lanes 4g + t of region (h, ab).
SLAI_HD int q6_ql_off(int r, int idx) {
    const int h = idx >> 6, i = idx & 63, c = i >> 4, pair = c >> 1, t = ((c & 1) << 1) | ((i >> 3) & 1), g = r & 7, ab = r >> 3;
    return ((h * 2 + pair) * 2 + ab) * 256 + (4 * g + t) * 8 + (i & 7);
}
SLAI_HD int q6_qh_off(int r, int idx) {
    const int h = idx >> 5, i = idx & 31, g = r & 7, ab = r >> 3;
    return 2048 + (h * 2 + ab) * 256 + (4 * g + (i >> 3)) * 8 + (i & 7);
}

// Copy GGUF block number `blk` of row `row` (raw bytes at `src`) to its place in the tile-major matrix.
SLAI_HD void place_block(int fmt, const uint8_t* src, uint8_t* data, int64_t row, int64_t blk, int64_t K) {
    const int64_t tile = row >> 4;
    const int r = (int)(row & 15);
    const int64_t ns = num_steps(fmt, K);
    if (fmt == 8) {
        const int64_t step = blk >> 2;
        const int b = (int)(blk & 3);
        uint8_t* d = data + (tile * ns + step) * 2176;
        d[8 * r + 2 * b] = src[0];
        d[8 * r + 2 * b + 1] = src[1];
        for (int i = 0; i < 32; i++) d[qbyte_off(128, r, 32 * b + i)] = src[2 + i];
        return;
    }
    uint8_t* d = data + (tile * ns + blk) * step_bytes(fmt);
    if (fmt == 12 || fmt == 13) {
        uint8_t* h = d + K45_HDR_ROW * r;
        for (int i = 0; i < 4; i++) h[i] = src[i];
        const uint32_t s0 = src[4] | (src[5] << 8) | (src[6] << 16) | ((uint32_t)src[7] << 24);
        const uint32_t s1 = src[8] | (src[9] << 8) | (src[10] << 16) | ((uint32_t)src[11] << 24);
        const uint32_t s2 = src[12] | (src[13] << 8) | (src[14] << 16) | ((uint32_t)src[15] << 24);
        for (int j = 0; j < 8; j++) {
            uint32_t sc, m;
            frag::scale_min_k4(j, s0, s1, s2, sc, m);
            h[k45_sc_off(j)] = (uint8_t)sc;
            h[12 + j] = (uint8_t)m;
        }
        if (fmt == 12) {
            for (int i = 0; i < 128; i++) d[qbyte_off(K45_HDR, r, i)] = src[16 + i];
        } else {
            for (int i = 0; i < 32; i++) d[K45_HDR + 32 * r + i] = src[16 + i];
            for (int i = 0; i < 128; i++) d[qbyte_off(K45_HDR + 512, r, i)] = src[48 + i];
        }
    } else if (fmt == 14) {
        for (int i = 0; i < 128; i++) d[q6_ql_off(r, i)] = src[i];
        for (int i = 0; i < 64; i++) d[q6_qh_off(r, i)] = src[128 + i];
        for (int i = 0; i < 16; i++) d[3072 + 16 * r + i] = src[192 + i];
        d[3328 + 2 * r] = src[208];
        d[3328 + 2 * r + 1] = src[209];
    }
}

}  // namespace layout
