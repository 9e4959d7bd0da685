// TEST INFRASTRUCTURE — CPU oracle for the slai decode hot path.
//
// This file restates, in plain C++, the CPU operator path of dimforge/slai (Rust) that the
// CUDA library is checked against.  It is not part of the product: only the test-suite, the
// smoke check and the benchmark's CPU-baseline legs may load it.  The reference is Rust and
// cannot be compiled in this environment, so nothing here is generated from it; every
// function names the reference lines it follows.
//
// Parity pinning: the reference stores no golden vectors for this path.  The oracle is pinned
// against (1) the deterministic block recipes of the reference's disabled dequantisation test
// (crates/slai/src/ops/quantization.rs:77-221) whose expected values are
// `Block*::dequantize()`, and (2) an independent dequantiser (python `gguf.quants`) when it is
// installed.  GEMV / attention / model-level results have no pin in the reference's own tests:
// for those rows parity is "unpinned" and rests on this restatement alone.
//
// Build: g++ -O2 -ffp-contract=off (no FMA contraction: `d*sc*q - dmin*m` must round exactly
// like the reference's separate f32 multiply / subtract).
//
// Summation order: nalgebra's `gemv`, `dot`, `norm_squared`, `mean` are restated as sequential
// f32 accumulation in index order (nalgebra 0.34 source is not in the reference tree, so the
// exact order is unpinned; `ora_gemv_f64acc` bounds the difference).

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>
#include <algorithm>

#define ORA_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------------------------
// f16 <-> f32.  decode follows crates/slai/src/quantization.rs:392-409 (exact IEEE binary16).
// ---------------------------------------------------------------------------------------------
ORA_API float ora_decode_f16(uint16_t half) {
    const uint16_t exp = (half >> 10) & 0x1f;
    const uint16_t mant = half & 0x3ff;
    float val;
    if (exp == 0) {
        val = (float)mant * std::ldexp(1.0f, -24);
    } else if (exp != 31) {
        val = ((float)mant + 1024.0f) * std::ldexp(1.0f, (int)exp - 25);
    } else if (mant == 0) {
        val = INFINITY;
    } else {
        val = NAN;
    }
    return (half & 0x8000) ? -val : val;
}

// Round-to-nearest-even f32 -> f16 (used only to model an fp16 KV cache; the reference keeps
// its cache in f32, crates/slai/src/models/llama2/transformer.rs:87-106).
ORA_API uint16_t ora_encode_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477ff000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x38800000u) {  // subnormal half (or zero)
        if (absx < 0x33000000u) return (uint16_t)sign;  // < 2^-25 -> 0
        const int e = (int)(absx >> 23);                // biased f32 exponent
        const uint32_t m = (absx & 0x7fffffu) | 0x800000u;
        const int shift = 126 - e;  // value = m * 2^(e-150); half subnormal unit 2^-24
        // result = round(m * 2^(e-150) / 2^-24) = round(m >> (126 - e))
        const uint32_t q = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1);
        uint32_t r = q;
        if (rem > halfway || (rem == halfway && (q & 1u))) r++;
        return (uint16_t)(sign | r);
    }
    // normal
    uint32_t r = ((absx - 0x38000000u) >> 13);
    const uint32_t rem = absx & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r++;
    return (uint16_t)(sign | r);
}

// ---------------------------------------------------------------------------------------------
// Block layouts (bytes exactly as in a GGUF file).
// ---------------------------------------------------------------------------------------------
enum { ORA_FMT_F32 = 0, ORA_FMT_Q8_0 = 8, ORA_FMT_Q4_K = 12, ORA_FMT_Q5_K = 13, ORA_FMT_Q6_K = 14 };

static const int QK_K = 256;

#pragma pack(push, 1)
struct BlockQ8_0 {  // quantization.rs:29-32
    uint16_t scale;
    int8_t data[32];
};
struct BlockQ4K {  // quantization.rs:322-327
    uint16_t d, dmin;
    uint8_t scales[12];
    uint8_t qs[128];
};
struct BlockQ5K {  // quantization.rs:249-255
    uint16_t d, dmin;
    uint8_t scales[12];
    uint8_t qh[32];
    uint8_t qs[128];
};
struct BlockQ6K {  // quantization.rs:204-209
    uint8_t ql[128];
    uint8_t qh[64];
    int8_t scales[16];
    uint16_t d;
};
#pragma pack(pop)
static_assert(sizeof(BlockQ8_0) == 34, "");
static_assert(sizeof(BlockQ4K) == 144, "");
static_assert(sizeof(BlockQ5K) == 176, "");
static_assert(sizeof(BlockQ6K) == 210, "");

// quantization.rs:381-389
static inline void get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (uint8_t)((q[j + 4] & 0xf) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// quantization.rs:38-41
static void dequant_q8_0(const BlockQ8_0* b, float* out) {
    const float scale = ora_decode_f16(b->scale);
    for (int i = 0; i < 32; i++) out[i] = (float)b->data[i] * scale;
}

// quantization.rs:347-378
static void dequant_q4k(const BlockQ4K* b, float* out) {
    const float d = ora_decode_f16(b->d);
    const float mn = ora_decode_f16(b->dmin);
    int is = 0, iq = 0;
    uint8_t sc = 0, m = 0;
    for (int j = 0; j < QK_K; j += 64) {
        get_scale_min_k4(is, b->scales, &sc, &m);
        const float d1 = d * (float)sc;
        const float m1 = mn * (float)m;
        get_scale_min_k4(is + 1, b->scales, &sc, &m);
        const float d2 = d * (float)sc;
        const float m2 = mn * (float)m;
        for (int l = 0; l < 32; l++) out[j + l] = d1 * (float)(b->qs[iq + l] & 0xF) - m1;
        for (int l = 0; l < 32; l++) out[j + l + 32] = d2 * (float)(b->qs[iq + l] >> 4) - m2;
        iq += 32;
        is += 2;
    }
}

// quantization.rs:275-316
static void dequant_q5k(const BlockQ5K* b, float* out) {
    const float d = ora_decode_f16(b->d);
    const float mn = ora_decode_f16(b->dmin);
    int is = 0, iq = 0;
    uint8_t sc = 0, m = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int j = 0; j < QK_K; j += 64) {
        get_scale_min_k4(is, b->scales, &sc, &m);
        const float d1 = d * (float)sc;
        const float m1 = mn * (float)m;
        get_scale_min_k4(is + 1, b->scales, &sc, &m);
        const float d2 = d * (float)sc;
        const float m2 = mn * (float)m;
        for (int l = 0; l < 32; l++) {
            const uint8_t q = (uint8_t)((b->qs[iq + l] & 0xF) + ((b->qh[l] & u1) ? 16 : 0));
            out[j + l] = d1 * (float)q - m1;
        }
        for (int l = 0; l < 32; l++) {
            const uint8_t q = (uint8_t)((b->qs[iq + l] >> 4) + ((b->qh[l] & u2) ? 16 : 0));
            out[j + l + 32] = d2 * (float)q - m2;
        }
        iq += 32;
        is += 2;
        u1 = (uint8_t)(u1 << 2);
        u2 = (uint8_t)(u2 << 2);
    }
}

// quantization.rs:214-243   (Rust evaluates `d * scale as f32 * q as f32` left to right)
static void dequant_q6k(const BlockQ6K* b, float* out) {
    const float d = ora_decode_f16(b->d);
    for (int i = 0; i < 2; i++) {
        for (int l = 0; l < 32; l++) {
            const int is = l / 16;
            const uint8_t ql0 = b->ql[i * 64 + l];
            const uint8_t ql32 = b->ql[i * 64 + l + 32];
            const uint8_t qh = b->qh[i * 32 + l];
            const int8_t q1 = (int8_t)((ql0 & 0xF) | (((qh >> 0) & 3) << 4)) - 32;
            const int8_t q2 = (int8_t)((ql32 & 0xF) | (((qh >> 2) & 3) << 4)) - 32;
            const int8_t q3 = (int8_t)((ql0 >> 4) | (((qh >> 4) & 3) << 4)) - 32;
            const int8_t q4 = (int8_t)((ql32 >> 4) | (((qh >> 6) & 3) << 4)) - 32;
            out[i * 128 + l + 0] = d * (float)b->scales[i * 8 + is + 0] * (float)q1;
            out[i * 128 + l + 32] = d * (float)b->scales[i * 8 + is + 2] * (float)q2;
            out[i * 128 + l + 64] = d * (float)b->scales[i * 8 + is + 4] * (float)q3;
            out[i * 128 + l + 96] = d * (float)b->scales[i * 8 + is + 6] * (float)q4;
        }
    }
}

ORA_API int ora_block_bytes(int fmt) {
    switch (fmt) {
        case ORA_FMT_F32: return 4;
        case ORA_FMT_Q8_0: return 34;
        case ORA_FMT_Q4_K: return 144;
        case ORA_FMT_Q5_K: return 176;
        case ORA_FMT_Q6_K: return 210;
    }
    return -1;
}
ORA_API int ora_block_elems(int fmt) {
    switch (fmt) {
        case ORA_FMT_F32: return 1;
        case ORA_FMT_Q8_0: return 32;
        case ORA_FMT_Q4_K:
        case ORA_FMT_Q5_K:
        case ORA_FMT_Q6_K: return 256;
    }
    return -1;
}

// ---- legacy 32-element formats and Q8_K (crates/slai/src/quantization.rs:47-199) -------------------------------
// Q4_0 (:47-70): f16 d, 16 bytes; element j = low nibble of qs[j] - 8, element j + 16 = high nibble - 8; times d.
static void dequant_q4_0(const uint8_t* b, float* out) {
    const float d = ora_decode_f16((uint16_t)(b[0] | (b[1] << 8)));
    for (int j = 0; j < 16; j++) {
        const int x0 = (int)(b[2 + j] & 0x0F) - 8, x1 = (int)(b[2 + j] >> 4) - 8;
        out[j] = (float)x0 * d;
        out[j + 16] = (float)x1 * d;
    }
}
// Q4_1 (:72-98): f16 d, f16 m, 16 bytes; nibble * d + m.
static void dequant_q4_1(const uint8_t* b, float* out) {
    const float d = ora_decode_f16((uint16_t)(b[0] | (b[1] << 8))), m = ora_decode_f16((uint16_t)(b[2] | (b[3] << 8)));
    for (int j = 0; j < 16; j++) {
        out[j] = (float)(b[4 + j] & 0x0F) * d + m;
        out[j + 16] = (float)(b[4 + j] >> 4) * d + m;
    }
}
// Q5_0 (:100-129): f16 d, 4 bytes of fifth bits (bit j for element j, bit j + 16 for element j + 16), 16 bytes; (q - 16) * d.
static void dequant_q5_0(const uint8_t* b, float* out) {
    const float d = ora_decode_f16((uint16_t)(b[0] | (b[1] << 8)));
    const uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
    for (int j = 0; j < 16; j++) {
        const uint32_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
        const int x0 = (int)(((uint32_t)b[6 + j] & 0x0F) | xh0) - 16, x1 = (int)(((uint32_t)b[6 + j] >> 4) | xh1) - 16;
        out[j] = (float)x0 * d;
        out[j + 16] = (float)x1 * d;
    }
}
// Q5_1 (:131-163): f16 d, f16 m, fifth bits, 16 bytes; q * d + m.
static void dequant_q5_1(const uint8_t* b, float* out) {
    const float d = ora_decode_f16((uint16_t)(b[0] | (b[1] << 8))), m = ora_decode_f16((uint16_t)(b[2] | (b[3] << 8)));
    const uint32_t qh = (uint32_t)b[4] | ((uint32_t)b[5] << 8) | ((uint32_t)b[6] << 16) | ((uint32_t)b[7] << 24);
    for (int j = 0; j < 16; j++) {
        const uint32_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
        out[j] = (float)(((uint32_t)b[8 + j] & 0x0F) | xh0) * d + m;
        out[j + 16] = (float)(((uint32_t)b[8 + j] >> 4) | xh1) * d + m;
    }
}
// Q8_K (:168-199): f32 d, 256 int8, 16 i16 group sums (unused by the dequantiser); d * q.
static void dequant_q8_k(const uint8_t* b, float* out) {
    float d;
    std::memcpy(&d, b, 4);
    for (int j = 0; j < 256; j++) out[j] = d * (float)(int8_t)b[4 + j];
}

// Dequantise `nblocks` consecutive blocks (a GGUF tensor is rows of blocks in row-major order,
// crates/slai/src/gguf.rs:116-131,596-676).  Returns 0 on success.
ORA_API int ora_dequantize(int fmt, const void* blocks, int64_t nblocks, float* out) {
    const uint8_t* p = (const uint8_t*)blocks;
    switch (fmt) {
        case ORA_FMT_F32: std::memcpy(out, blocks, (size_t)nblocks * 4); return 0;
        case ORA_FMT_Q8_0:
            for (int64_t i = 0; i < nblocks; i++) dequant_q8_0((const BlockQ8_0*)(p + i * 34), out + i * 32);
            return 0;
        case ORA_FMT_Q4_K:
            for (int64_t i = 0; i < nblocks; i++) dequant_q4k((const BlockQ4K*)(p + i * 144), out + i * 256);
            return 0;
        case ORA_FMT_Q5_K:
            for (int64_t i = 0; i < nblocks; i++) dequant_q5k((const BlockQ5K*)(p + i * 176), out + i * 256);
            return 0;
        case ORA_FMT_Q6_K:
            for (int64_t i = 0; i < nblocks; i++) dequant_q6k((const BlockQ6K*)(p + i * 210), out + i * 256);
            return 0;
        case 2:
            for (int64_t i = 0; i < nblocks; i++) dequant_q4_0(p + i * 18, out + i * 32);
            return 0;
        case 3:
            for (int64_t i = 0; i < nblocks; i++) dequant_q4_1(p + i * 20, out + i * 32);
            return 0;
        case 6:
            for (int64_t i = 0; i < nblocks; i++) dequant_q5_0(p + i * 22, out + i * 32);
            return 0;
        case 7:
            for (int64_t i = 0; i < nblocks; i++) dequant_q5_1(p + i * 24, out + i * 32);
            return 0;
        case 15:
            for (int64_t i = 0; i < nblocks; i++) dequant_q8_k(p + i * 292, out + i * 256);
            return 0;
    }
    return -1;
}

// ---------------------------------------------------------------------------------------------
// Dense f32 GEMV: the reference CPU path dequantises every weight at load and calls nalgebra
// `out.gemv(1.0, w, x, 0.0)` (crates/slai/src/models/llama2/cpu.rs:200-219,370-376).
// `w` is row-major M x K here.  Rows are partitioned over `nthreads` (the reference is
// single-threaded; the threaded form is used only for the all-core timing).
// ---------------------------------------------------------------------------------------------
static void gemv_rows(float* out, const float* w, const float* x, int64_t r0, int64_t r1, int64_t K) {
    for (int64_t i = r0; i < r1; i++) {
        const float* wr = w + i * K;
        float acc = 0.0f;
        for (int64_t j = 0; j < K; j++) acc += wr[j] * x[j];
        out[i] = acc;
    }
}

template <class F>
static void parallel_rows(int64_t M, int nthreads, F f) {
    if (nthreads <= 1 || M < 2 * nthreads) {
        f(0, M);
        return;
    }
    std::vector<std::thread> th;
    const int64_t per = (M + nthreads - 1) / nthreads;
    for (int t = 0; t < nthreads; t++) {
        const int64_t r0 = t * per, r1 = std::min<int64_t>(M, r0 + per);
        if (r0 >= r1) break;
        th.emplace_back([=] { f(r0, r1); });
    }
    for (auto& t : th) t.join();
}

ORA_API void ora_gemv_f32(float* out, const float* w, const float* x, int64_t M, int64_t K, int nthreads) {
    parallel_rows(M, nthreads, [=](int64_t r0, int64_t r1) { gemv_rows(out, w, x, r0, r1, K); });
}

// Same product accumulated in f64 (bounds the effect of the unpinned f32 summation order).
ORA_API void ora_gemv_f64acc(float* out, const float* w, const float* x, int64_t M, int64_t K) {
    for (int64_t i = 0; i < M; i++) {
        double acc = 0.0;
        for (int64_t j = 0; j < K; j++) acc += (double)w[i * K + j] * (double)x[j];
        out[i] = (float)acc;
    }
}

// Quantised GEMV on the CPU = dequantise, then dense GEMV (what `GemvQuant` must equal:
// crates/slai/src/ops/gemv_quant.rs:206-312 computes out = m * v on dequantised values).
ORA_API int ora_gemv_quant(int fmt, float* out, const void* blocks, const float* x, int64_t M, int64_t K,
                           int nthreads) {
    const int be = ora_block_elems(fmt), bb = ora_block_bytes(fmt);
    if (be <= 0 || K % be != 0) return -1;
    const int64_t row_bytes = K / be * bb;
    parallel_rows(M, nthreads, [=](int64_t r0, int64_t r1) {
        std::vector<float> row((size_t)K);
        for (int64_t i = r0; i < r1; i++) {
            ora_dequantize(fmt, (const uint8_t*)blocks + i * row_bytes, K / be, row.data());
            float acc = 0.0f;
            for (int64_t j = 0; j < K; j++) acc += row[j] * x[j];
            out[i] = acc;
        }
    });
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Element-wise / normalisation operators (the `run_cpu` twins).
// ---------------------------------------------------------------------------------------------

// crates/slai/src/ops/rms_norm.rs:68-77 and models/llama2/cpu.rs:340-348 (eps is 1e-5 there;
// a parameter here).
ORA_API void ora_rms_norm(float* out, const float* a, const float* w, int64_t n, float eps) {
    float ss = 0.0f;
    for (int64_t i = 0; i < n; i++) ss += a[i] * a[i];
    const float rms = 1.0f / std::sqrt(ss / (float)n + eps);
    for (int64_t i = 0; i < n; i++) out[i] = (a[i] * rms) * w[i];
}

// crates/slai/src/ops/layernorm.rs:104-111 (no gamma/beta; caller applies them,
// models/gpt2/cpu.rs:235-240).
ORA_API void ora_layernorm(float* res, const float* v, int64_t n, float eps) {
    float sum = 0.0f;
    for (int64_t i = 0; i < n; i++) sum += v[i];
    const float mean = sum / (float)n;
    float ss = 0.0f;
    for (int64_t i = 0; i < n; i++) {
        res[i] = v[i] - mean;
        ss += res[i] * res[i];
    }
    const float variance = ss / (float)n;
    const float scale = 1.0f / std::sqrt(variance + eps);
    for (int64_t i = 0; i < n; i++) res[i] *= scale;
}

// crates/slai/src/ops/softmax.rs:46-59, models/llama2/cpu.rs:354-367
ORA_API void ora_softmax(float* vals, int64_t n) {
    float mx = vals[0];
    for (int64_t i = 1; i < n; i++) mx = std::max(mx, vals[i]);
    float sum = 0.0f;
    for (int64_t i = 0; i < n; i++) {
        vals[i] = std::exp(vals[i] - mx);
        sum += vals[i];
    }
    for (int64_t i = 0; i < n; i++) vals[i] /= sum;
}

// crates/slai/src/ops/silu.rs:50-58
ORA_API void ora_silu_gate(float* h1, const float* h2, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        const float x = h1[i];
        h1[i] = h2[i] * (x / (1.0f + std::exp(-1.0f * x)));
    }
}

// crates/slai/src/ops/unary.rs:11-35 (enum order) and :62-106 (eval)
enum {
    U_ABS, U_SGN, U_NEG, U_STEP, U_ELU, U_GELU, U_GELU_QUICK, U_SILU, U_TANH, U_SIN, U_COS, U_RELU,
    U_SIGMOID, U_HARD_SIGMOID, U_SQR, U_SQRT, U_LOG, U_LEAKY_RELU, U_CLAMP, U_SCALE, U_ADD_SCALAR
};
static float unary_eval(int op, float x, const float* a) {
    switch (op) {
        case U_ABS: return std::fabs(x);
        case U_SGN: return std::isnan(x) ? x : std::copysign(1.0f, x);  // Rust f32::signum
        case U_NEG: return -x;
        case U_STEP: return x > 0.0f ? 1.0f : 0.0f;
        case U_ELU: return x > 0.0f ? x : std::exp(x) - 1.0f;
        case U_GELU: {
            const float A = 0.044715f, S = 0.7978846f;
            return 0.5f * x * (1.0f + std::tanh(S * x * (1.0f + A * x * x)));
        }
        case U_GELU_QUICK: return x * (1.0f / (1.0f + std::exp(-1.702f * x)));
        case U_SILU: return x / (1.0f + std::exp(-x));
        case U_TANH: return std::tanh(x);
        case U_SIN: return std::sin(x);
        case U_COS: return std::cos(x);
        case U_RELU: return std::max(x, 0.0f);
        case U_SIGMOID: return 1.0f / (1.0f + std::exp(-x));
        case U_HARD_SIGMOID: return std::min(1.0f, std::max(0.0f, (x + 3.0f) / 6.0f));
        case U_SQR: return x * x;
        case U_SQRT: return std::sqrt(x);
        case U_LOG: return std::log(x);
        case U_LEAKY_RELU: return std::max(x, 0.0f) + std::min(x, 0.0f) * a[0];
        case U_CLAMP: return std::min(std::max(x, a[0]), a[1]);
        case U_SCALE: return x * a[0];
        case U_ADD_SCALAR: return x + a[0];
    }
    return NAN;
}
ORA_API void ora_unary(int op, float* dst, const float* src, int64_t n, const float* args4) {
    for (int64_t i = 0; i < n; i++) dst[i] = unary_eval(op, src[i], args4);
}

// crates/slai/src/ops/rope.rs:88-125 (adjacent pairs; base is hard-coded 10000 in the CPU twin,
// a parameter here as in RoPEConfig :28-33) and shaders/slai/rope.slang:58-86 for the NeoX
// pairing (element `i + head*hs/2` with the one `hs/2` further on).
ORA_API void ora_rope(int neox, float* q, float* k, int head_size, int dim, int kv_dim, int pos, float base) {
    for (int i = 0; i < dim; i += 2) {
        const float head_dim = (float)(i % head_size);
        const float theta = std::pow(base, -head_dim / (float)head_size);
        const float m_theta = (float)pos * theta;
        const float c = std::cos(m_theta), s = std::sin(m_theta);
        int i0, i1;
        if (!neox) {
            i0 = i;
            i1 = i + 1;
        } else {
            const int pair = i / 2;
            const int head_id = i / head_size;
            i0 = pair + head_id * head_size / 2;
            i1 = i0 + head_size / 2;
        }
        const float q0 = q[i0], q1 = q[i1];
        q[i0] = c * q0 - s * q1;
        q[i1] = s * q0 + c * q1;
        if (i < kv_dim) {
            const float k0 = k[i0], k1 = k[i1];
            k[i0] = c * k0 - s * k1;
            k[i1] = s * k0 + c * k1;
        }
    }
}

// crates/slai/src/ops/batched_multiquery_attention.rs:102-156.  Caches are position-major:
// position t occupies kv_dim consecutive floats (a column of the reference's DMatrix).
// `att` is n_heads columns of seq_len floats.
ORA_API void ora_attention(int seq_len, int kv_dim, int kv_mul, int n_heads, int head_size, int pos,
                           const float* q, const float* key_cache, const float* value_cache, float* att,
                           float* xb) {
    for (int h = 0; h < n_heads; h++) {
        const float* qh = q + (size_t)h * head_size;
        float* a = att + (size_t)h * seq_len;
        for (int t = 0; t <= pos; t++) {
            const float* kh = key_cache + (size_t)t * kv_dim + (size_t)(h / kv_mul) * head_size;
            float score = 0.0f;
            for (int i = 0; i < head_size; i++) score += qh[i] * kh[i];
            score /= std::sqrt((float)head_size);
            a[t] = score;
        }
        ora_softmax(a, pos + 1);
        float* o = xb + (size_t)h * head_size;
        for (int i = 0; i < head_size; i++) o[i] = 0.0f;
        for (int t = 0; t <= pos; t++) {
            const float* vh = value_cache + (size_t)t * kv_dim + (size_t)(h / kv_mul) * head_size;
            const float w = a[t];
            for (int i = 0; i < head_size; i++) o[i] += w * vh[i];
        }
    }
}

// crates/slai/src/models/sampler.rs:34-36,55-57: greedy = nalgebra `imax` (first maximal index).
ORA_API int ora_argmax(const float* v, int64_t n) {
    int64_t best = 0;
    for (int64_t i = 1; i < n; i++)
        if (v[i] > v[best]) best = i;
    return (int)best;
}

// crates/slai/src/models/sampler.rs:33-131: temperature, softmax, then either a draw from the whole distribution
// (sample_mult, :63-78) or nucleus sampling (sample_topp, :85-131: candidates >= (1 - topp) / (n - 1), stable sort by
// descending probability, truncation where the cumulative probability exceeds topp, draw inside the truncated
// list).  The reference draws `coin` from an unseeded generator (:43); here it is an argument.  `logits` is
// overwritten with the probabilities, as in the reference.
ORA_API int ora_sample(float* logits, int64_t n, float temperature, float topp, float coin) {
    if (temperature == 0.0f) return ora_argmax(logits, n);
    for (int64_t i = 0; i < n; i++) logits[i] /= temperature;
    ora_softmax(logits, n);
    if (topp <= 0.0f || topp >= 1.0f) {
        float cdf = 0.0f;
        for (int64_t i = 0; i < n; i++) {
            cdf += logits[i];
            if (coin < cdf) return (int)i;
        }
        return (int)(n - 1);
    }
    const float cutoff = (1.0f - topp) / ((float)n - 1.0f);
    std::vector<std::pair<float, int>> cand;
    for (int64_t i = 0; i < n; i++)
        if (logits[i] >= cutoff) cand.push_back({logits[i], (int)i});
    std::stable_sort(cand.begin(), cand.end(), [](const std::pair<float, int>& a, const std::pair<float, int>& b) { return a.first > b.first; });
    const int n0 = (int)cand.size();
    if (n0 == 0) {  // the reference panics on `n0 - 1` here; defined as the greedy choice (first maximal index, else 0)
        int best = 0;
        float bv = -INFINITY;
        bool any = false;
        for (int64_t i = 0; i < n; i++)
            if (logits[i] > bv) {
                bv = logits[i];
                best = (int)i;
                any = true;
            }
        return any ? best : 0;
    }
    float cumulative = 0.0f;
    int last = n0 - 1;
    for (int i = 0; i < n0; i++) {
        cumulative += cand[i].first;
        if (cumulative > topp) {
            last = i;
            break;
        }
    }
    const float r = coin * cumulative;
    float cdf = 0.0f;
    for (int i = 0; i <= last; i++) {
        cdf += cand[i].first;
        if (r < cdf) return cand[i].second;
    }
    return cand[last].second;
}

// ---------------------------------------------------------------------------------------------
// Models: dense f32 weights supplied by the caller (already dequantised, as the reference does
// at load: models/llama2/cpu.rs:200-219; models/gpt2/cpu.rs:113-217).
// ---------------------------------------------------------------------------------------------
struct OraLlamaLayer {
    const float *attn_norm, *wq, *wk, *wv, *wo, *ffn_norm, *w_gate, *w_up, *w_down;
    const float *bq, *bk, *bv;  // optional biases (Qwen2; transformer.rs:336-344)
};
struct OraLlama {
    int dim, hidden, n_layers, n_q, n_kv, vocab, seq_len;
    float rope_base, eps;
    int neox, kv_f16, nthreads;
    std::vector<OraLlamaLayer> layers;
    const float *token_embd, *out_norm, *w_out;  // token_embd: vocab rows of dim floats
    std::vector<float> x, xb, xb2, hb, hb2, q, att, logits;
    std::vector<std::vector<float>> kc, vc;  // per layer: seq_len x kv_dim
};

ORA_API OraLlama* ora_llama_create(int dim, int hidden, int n_layers, int n_q, int n_kv, int vocab, int seq_len,
                                   float rope_base, float eps, int neox, int kv_f16, int nthreads) {
    OraLlama* m = new OraLlama();
    m->dim = dim; m->hidden = hidden; m->n_layers = n_layers; m->n_q = n_q; m->n_kv = n_kv;
    m->vocab = vocab; m->seq_len = seq_len; m->rope_base = rope_base; m->eps = eps;
    m->neox = neox; m->kv_f16 = kv_f16; m->nthreads = nthreads;
    m->layers.resize(n_layers);
    for (auto& l : m->layers) std::memset(&l, 0, sizeof(l));
    const int kv_dim = dim * n_kv / n_q;
    m->x.resize(dim); m->xb.resize(dim); m->xb2.resize(dim); m->q.resize(dim);
    m->hb.resize(hidden); m->hb2.resize(hidden);
    m->att.resize((size_t)seq_len * n_q); m->logits.resize(vocab);
    m->kc.assign(n_layers, std::vector<float>((size_t)seq_len * kv_dim));
    m->vc.assign(n_layers, std::vector<float>((size_t)seq_len * kv_dim));
    m->token_embd = m->out_norm = m->w_out = nullptr;
    return m;
}
ORA_API void ora_llama_destroy(OraLlama* m) { delete m; }

// Weight ids shared with the CUDA library's header.
enum {
    W_TOKEN_EMBD = 0, W_OUT_NORM = 1, W_OUTPUT = 2, W_ATTN_NORM = 3, W_Q = 4, W_K = 5, W_V = 6, W_O = 7,
    W_FFN_NORM = 8, W_GATE = 9, W_UP = 10, W_DOWN = 11, W_BQ = 12, W_BK = 13, W_BV = 14
};
ORA_API int ora_llama_set_weight(OraLlama* m, int id, int layer, const float* p) {
    if (id <= W_OUTPUT) {
        if (id == W_TOKEN_EMBD) m->token_embd = p;
        else if (id == W_OUT_NORM) m->out_norm = p;
        else m->w_out = p;
        return 0;
    }
    if (layer < 0 || layer >= m->n_layers) return -1;
    OraLlamaLayer& l = m->layers[layer];
    switch (id) {
        case W_ATTN_NORM: l.attn_norm = p; break;
        case W_Q: l.wq = p; break;
        case W_K: l.wk = p; break;
        case W_V: l.wv = p; break;
        case W_O: l.wo = p; break;
        case W_FFN_NORM: l.ffn_norm = p; break;
        case W_GATE: l.w_gate = p; break;
        case W_UP: l.w_up = p; break;
        case W_DOWN: l.w_down = p; break;
        case W_BQ: l.bq = p; break;
        case W_BK: l.bk = p; break;
        case W_BV: l.bv = p; break;
        default: return -1;
    }
    return 0;
}

static void round_f16_inplace(float* v, int64_t n) {
    for (int64_t i = 0; i < n; i++) v[i] = ora_decode_f16(ora_encode_f16(v[i]));
}

// crates/slai/src/models/llama2/cpu.rs:379-446 (forward), :488-543 (attention), :545-564 (ffn).
ORA_API const float* ora_llama_forward(OraLlama* m, int token, int pos) {
    const int dim = m->dim, kv_dim = dim * m->n_kv / m->n_q, hs = dim / m->n_q, kv_mul = m->n_q / m->n_kv;
    const int nt = m->nthreads;
    std::memcpy(m->x.data(), m->token_embd + (size_t)token * dim, (size_t)dim * 4);
    for (int l = 0; l < m->n_layers; l++) {
        const OraLlamaLayer& w = m->layers[l];
        ora_rms_norm(m->xb.data(), m->x.data(), w.attn_norm, dim, m->eps);
        float* kcol = m->kc[l].data() + (size_t)pos * kv_dim;
        float* vcol = m->vc[l].data() + (size_t)pos * kv_dim;
        ora_gemv_f32(m->q.data(), w.wq, m->xb.data(), dim, dim, nt);
        ora_gemv_f32(kcol, w.wk, m->xb.data(), kv_dim, dim, nt);
        ora_gemv_f32(vcol, w.wv, m->xb.data(), kv_dim, dim, nt);
        if (w.bq) for (int i = 0; i < dim; i++) m->q[i] += w.bq[i];
        if (w.bk) for (int i = 0; i < kv_dim; i++) kcol[i] += w.bk[i];
        if (w.bv) for (int i = 0; i < kv_dim; i++) vcol[i] += w.bv[i];
        ora_rope(m->neox, m->q.data(), kcol, hs, dim, kv_dim, pos, m->rope_base);
        if (m->kv_f16) {
            round_f16_inplace(kcol, kv_dim);
            round_f16_inplace(vcol, kv_dim);
        }
        ora_attention(m->seq_len, kv_dim, kv_mul, m->n_q, hs, pos, m->q.data(), m->kc[l].data(),
                      m->vc[l].data(), m->att.data(), m->xb.data());
        ora_gemv_f32(m->xb2.data(), w.wo, m->xb.data(), dim, dim, nt);
        for (int i = 0; i < dim; i++) m->x[i] += m->xb2[i];
        ora_rms_norm(m->xb.data(), m->x.data(), w.ffn_norm, dim, m->eps);
        ora_gemv_f32(m->hb.data(), w.w_gate, m->xb.data(), m->hidden, dim, nt);
        ora_gemv_f32(m->hb2.data(), w.w_up, m->xb.data(), m->hidden, dim, nt);
        ora_silu_gate(m->hb.data(), m->hb2.data(), m->hidden);
        ora_gemv_f32(m->xb2.data(), w.w_down, m->hb.data(), dim, m->hidden, nt);
        for (int i = 0; i < dim; i++) m->x[i] += m->xb2[i];
    }
    ora_rms_norm(m->xb.data(), m->x.data(), m->out_norm, dim, m->eps);
    ora_gemv_f32(m->logits.data(), m->w_out, m->xb.data(), m->vocab, dim, nt);
    return m->logits.data();
}
ORA_API const float* ora_llama_x(OraLlama* m) { return m->x.data(); }

// GPT-2 ---------------------------------------------------------------------------------------
struct OraGpt2Layer {
    const float *ln1_g, *ln1_b, *w_qkv, *b_qkv, *w_proj, *b_proj, *ln2_g, *ln2_b, *w_fc, *b_fc, *w_fcproj, *b_fcproj;
};
struct OraGpt2 {
    int n_vocab, n_seq, n_embd, n_head, n_layer, ff_len;
    float eps;
    int kv_f16, nthreads;
    const float *wte, *wpe, *lnf_g, *lnf_b;  // wte: n_vocab rows of n_embd (also the tied lm_head)
    std::vector<OraGpt2Layer> layers;
    std::vector<float> x, cur, cur_b, qkv, q, ff, att, logits;
    std::vector<std::vector<float>> kc, vc;
};
enum {
    G_WTE = 0, G_WPE = 1, G_LNF_G = 2, G_LNF_B = 3, G_LN1_G = 4, G_LN1_B = 5, G_W_QKV = 6, G_B_QKV = 7,
    G_W_PROJ = 8, G_B_PROJ = 9, G_LN2_G = 10, G_LN2_B = 11, G_W_FC = 12, G_B_FC = 13, G_W_FCPROJ = 14,
    G_B_FCPROJ = 15
};
ORA_API OraGpt2* ora_gpt2_create(int n_vocab, int n_seq, int n_embd, int n_head, int n_layer, int ff_len,
                                 float eps, int kv_f16, int nthreads) {
    OraGpt2* m = new OraGpt2();
    m->n_vocab = n_vocab; m->n_seq = n_seq; m->n_embd = n_embd; m->n_head = n_head; m->n_layer = n_layer;
    m->ff_len = ff_len; m->eps = eps; m->kv_f16 = kv_f16; m->nthreads = nthreads;
    m->layers.resize(n_layer);
    for (auto& l : m->layers) std::memset(&l, 0, sizeof(l));
    m->x.resize(n_embd); m->cur.resize(n_embd); m->cur_b.resize(n_embd); m->q.resize(n_embd);
    m->qkv.resize(3 * (size_t)n_embd); m->ff.resize(ff_len);
    m->att.resize((size_t)n_seq * n_head); m->logits.resize(n_vocab);
    m->kc.assign(n_layer, std::vector<float>((size_t)n_seq * n_embd));
    m->vc.assign(n_layer, std::vector<float>((size_t)n_seq * n_embd));
    m->wte = m->wpe = m->lnf_g = m->lnf_b = nullptr;
    return m;
}
ORA_API void ora_gpt2_destroy(OraGpt2* m) { delete m; }
ORA_API int ora_gpt2_set_weight(OraGpt2* m, int id, int layer, const float* p) {
    switch (id) {
        case G_WTE: m->wte = p; return 0;
        case G_WPE: m->wpe = p; return 0;
        case G_LNF_G: m->lnf_g = p; return 0;
        case G_LNF_B: m->lnf_b = p; return 0;
    }
    if (layer < 0 || layer >= m->n_layer) return -1;
    OraGpt2Layer& l = m->layers[layer];
    switch (id) {
        case G_LN1_G: l.ln1_g = p; break;
        case G_LN1_B: l.ln1_b = p; break;
        case G_W_QKV: l.w_qkv = p; break;
        case G_B_QKV: l.b_qkv = p; break;
        case G_W_PROJ: l.w_proj = p; break;
        case G_B_PROJ: l.b_proj = p; break;
        case G_LN2_G: l.ln2_g = p; break;
        case G_LN2_B: l.ln2_b = p; break;
        case G_W_FC: l.w_fc = p; break;
        case G_B_FC: l.b_fc = p; break;
        case G_W_FCPROJ: l.w_fcproj = p; break;
        case G_B_FCPROJ: l.b_fcproj = p; break;
        default: return -1;
    }
    return 0;
}

static void ln_affine(float* out, const float* in, const float* g, const float* b, int n, float eps) {
    ora_layernorm(out, in, n, eps);
    for (int i = 0; i < n; i++) out[i] *= g[i];
    for (int i = 0; i < n; i++) out[i] += b[i];
}

// crates/slai/src/models/gpt2/cpu.rs:225-383
ORA_API const float* ora_gpt2_forward(OraGpt2* m, int token, int pos) {
    const int E = m->n_embd, nt = m->nthreads;
    for (int i = 0; i < E; i++) m->x[i] = m->wte[(size_t)token * E + i];
    for (int i = 0; i < E; i++) m->x[i] += m->wpe[(size_t)pos * E + i];
    for (int l = 0; l < m->n_layer; l++) {
        const OraGpt2Layer& w = m->layers[l];
        ln_affine(m->cur.data(), m->x.data(), w.ln1_g, w.ln1_b, E, m->eps);
        ora_gemv_f32(m->qkv.data(), w.w_qkv, m->cur.data(), 3 * E, E, nt);
        for (int i = 0; i < 3 * E; i++) m->qkv[i] += w.b_qkv[i];
        float* kcol = m->kc[l].data() + (size_t)pos * E;
        float* vcol = m->vc[l].data() + (size_t)pos * E;
        std::memcpy(m->q.data(), m->qkv.data(), (size_t)E * 4);
        std::memcpy(kcol, m->qkv.data() + E, (size_t)E * 4);
        std::memcpy(vcol, m->qkv.data() + 2 * E, (size_t)E * 4);
        if (m->kv_f16) {
            round_f16_inplace(kcol, E);
            round_f16_inplace(vcol, E);
        }
        ora_attention(m->n_seq, E, 1, m->n_head, E / m->n_head, pos, m->q.data(), m->kc[l].data(),
                      m->vc[l].data(), m->att.data(), m->cur.data());
        ora_gemv_f32(m->cur_b.data(), w.w_proj, m->cur.data(), E, E, nt);
        for (int i = 0; i < E; i++) m->cur_b[i] += w.b_proj[i];
        for (int i = 0; i < E; i++) m->cur_b[i] += m->x[i];
        std::memcpy(m->x.data(), m->cur_b.data(), (size_t)E * 4);
        ln_affine(m->cur.data(), m->cur_b.data(), w.ln2_g, w.ln2_b, E, m->eps);
        ora_gemv_f32(m->ff.data(), w.w_fc, m->cur.data(), m->ff_len, E, nt);
        for (int i = 0; i < m->ff_len; i++) m->ff[i] += w.b_fc[i];
        for (int i = 0; i < m->ff_len; i++) m->ff[i] = unary_eval(U_GELU, m->ff[i], nullptr);
        ora_gemv_f32(m->cur.data(), w.w_fcproj, m->ff.data(), E, m->ff_len, nt);
        for (int i = 0; i < E; i++) m->cur[i] += w.b_fcproj[i];
        for (int i = 0; i < E; i++) m->x[i] += m->cur[i];
    }
    ln_affine(m->cur.data(), m->x.data(), m->lnf_g, m->lnf_b, E, m->eps);
    ora_gemv_f32(m->logits.data(), m->wte, m->cur.data(), m->n_vocab, E, nt);
    return m->logits.data();
}

ORA_API int ora_hw_threads() { return (int)std::thread::hardware_concurrency(); }
