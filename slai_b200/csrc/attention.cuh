// Single-query attention over the KV cache, device side (see attention.cu for the operator).  Shared by the
// stand-alone attention kernel and the persistent decode kernel, which runs four items per block of threads.
#pragma once
#include "common.cuh"

namespace attn {

constexpr int ATT_THREADS = 128;
constexpr int ATT_WARPS = 4;
constexpr int MAX_J = 4;  // head_size <= 256

struct AttnParams {
    const float* q;
    const void* kc;
    const void* vc;
    long long pos_stride, head_stride;
    int n_heads, kv_mul, hs;
    const int* d_pos;
    int n_splits, chunk_max;
    float* out;
    float* part_o;   // [n_heads][n_splits][hs]
    float* part_ml;  // [n_heads][n_splits][2]
    unsigned int* counters;  // [n_kv_heads]
};

// Two consecutive cache elements as floats.  L2 loads (ld.global.cg): inside the persistent decode kernel the
// newest cache entry was written by another SM during the same launch, so L1 must not be trusted.
template <typename T> struct Ld2;
template <> struct Ld2<__half> {
    __device__ static float2 ld(const __half* p) {
        const unsigned int u = __ldcg(reinterpret_cast<const unsigned int*>(p));
        return __half22float2(*reinterpret_cast<const __half2*>(&u));
    }
};
template <> struct Ld2<float> {
    __device__ static float2 ld(const float* p) { return __ldcg(reinterpret_cast<const float2*>(p)); }
};

// Barrier over the ATT_THREADS threads that work on one item (named barrier `id`; id 0 with a 128-thread block is
// the block-wide barrier).
__device__ __forceinline__ void att_sync(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(ATT_THREADS) : "memory"); }

// Floats of shared memory one item needs.
__host__ __device__ inline size_t attn_item_floats(int kv_mul, int hs, int chunk_max) {
    return (size_t)kv_mul * hs + (size_t)kv_mul * chunk_max + (size_t)ATT_WARPS * kv_mul * hs + 2 * (size_t)kv_mul + 4;
}

// One work item = (KV head, split of the positions), processed by ATT_THREADS threads with thread index `tid`,
// shared memory `sm` (attn_item_floats floats) and barrier `bar_id`.
template <typename T, int MAXQ>
__device__ void attn_item(const AttnParams& P, int kvh, int split, int tid, float* sm, int bar_id) {
    const int hs = P.hs, kv_mul = P.kv_mul;
    float* q_s = sm;                                 // [kv_mul][hs]
    float* sc_s = q_s + kv_mul * hs;                 // [kv_mul][chunk_max]
    float* red_s = sc_s + kv_mul * P.chunk_max;      // [ATT_WARPS][kv_mul][hs]
    float* ml_s = red_s + ATT_WARPS * kv_mul * hs;   // [kv_mul][2]
    int* is_last_p = reinterpret_cast<int*>(ml_s + 2 * kv_mul);
    const int lane = tid & 31, warp = tid >> 5;

    const int n = __ldcg(P.d_pos) + 1;
    const int chunk = (n + P.n_splits - 1) / P.n_splits;
    const int t0 = split * chunk;
    const int t1 = min(n, t0 + chunk);
    const int cnt = max(0, t1 - t0);

    for (int i = tid; i < kv_mul * hs; i += ATT_THREADS) q_s[i] = __ldcg(P.q + (size_t)kvh * kv_mul * hs + i);
    att_sync(bar_id);

    const T* kbase = reinterpret_cast<const T*>(P.kc) + (size_t)kvh * P.head_stride;
    const T* vbase = reinterpret_cast<const T*>(P.vc) + (size_t)kvh * P.head_stride;
    const float inv_sqrt = sqrtf((float)hs);

    // Phase 1: scores.  Eight lanes per position, four positions per warp iteration.
    {
        const int sub = lane >> 3, l8 = lane & 7;
        for (int i0 = warp * 4; i0 < cnt; i0 += ATT_WARPS * 4) {
            const int i = i0 + sub;
            float part[MAXQ];
#pragma unroll
            for (int h = 0; h < MAXQ; h++) part[h] = 0.f;
            if (i < cnt) {
                const T* kp = kbase + (size_t)(t0 + i) * P.pos_stride;
                for (int e = l8; e < (hs >> 1); e += 8) {
                    const float2 k2 = Ld2<T>::ld(kp + 2 * e);
#pragma unroll
                    for (int h = 0; h < MAXQ; h++)
                        if (h < kv_mul) part[h] = fmaf(k2.y, q_s[h * hs + 2 * e + 1], fmaf(k2.x, q_s[h * hs + 2 * e], part[h]));
                }
            }
#pragma unroll
            for (int h = 0; h < MAXQ; h++) {
                part[h] += __shfl_xor_sync(0xffffffffu, part[h], 1);
                part[h] += __shfl_xor_sync(0xffffffffu, part[h], 2);
                part[h] += __shfl_xor_sync(0xffffffffu, part[h], 4);
            }
            if (i < cnt && l8 == 0) {
#pragma unroll
                for (int h = 0; h < MAXQ; h++)
                    if (h < kv_mul) sc_s[h * P.chunk_max + i] = part[h] / inv_sqrt;
            }
        }
    }
    att_sync(bar_id);
    // Phase 1b: local softmax numerators per query head.
    for (int h = warp; h < kv_mul; h += ATT_WARPS) {
        float m = -INFINITY;
        for (int i = lane; i < cnt; i += 32) m = fmaxf(m, sc_s[h * P.chunk_max + i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
        for (int i = lane; i < cnt; i += 32) {
            const float p = expf(sc_s[h * P.chunk_max + i] - m);
            sc_s[h * P.chunk_max + i] = p;
            l += p;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) {
            ml_s[2 * h] = m;
            ml_s[2 * h + 1] = l;
        }
    }
    att_sync(bar_id);
    // Phase 2: weighted sum of V.  A warp takes every ATT_WARPS-th position; a lane owns dims 64j+2*lane.
    float acc[MAXQ][MAX_J][2];
#pragma unroll
    for (int h = 0; h < MAXQ; h++)
#pragma unroll
        for (int j = 0; j < MAX_J; j++) acc[h][j][0] = acc[h][j][1] = 0.f;
    for (int i = warp; i < cnt; i += ATT_WARPS) {
        const T* vp = vbase + (size_t)(t0 + i) * P.pos_stride;
#pragma unroll
        for (int j = 0; j < MAX_J; j++) {
            const int d = 64 * j + 2 * lane;
            if (d < hs) {
                const float2 v2 = Ld2<T>::ld(vp + d);
#pragma unroll
                for (int h = 0; h < MAXQ; h++)
                    if (h < kv_mul) {
                        const float p = sc_s[h * P.chunk_max + i];
                        acc[h][j][0] = fmaf(p, v2.x, acc[h][j][0]);
                        acc[h][j][1] = fmaf(p, v2.y, acc[h][j][1]);
                    }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < MAXQ; h++)
        if (h < kv_mul)
#pragma unroll
            for (int j = 0; j < MAX_J; j++) {
                const int d = 64 * j + 2 * lane;
                if (d < hs) {
                    red_s[(warp * kv_mul + h) * hs + d] = acc[h][j][0];
                    red_s[(warp * kv_mul + h) * hs + d + 1] = acc[h][j][1];
                }
            }
    att_sync(bar_id);
    for (int i = tid; i < kv_mul * hs; i += ATT_THREADS) {
        const int h = i / hs, d = i % hs;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) o += red_s[(w * kv_mul + h) * hs + d];
        const int head = kvh * kv_mul + h;
        if (P.n_splits == 1) {
            P.out[(size_t)head * hs + d] = o / ml_s[2 * h + 1];
        } else {
            P.part_o[((size_t)head * P.n_splits + split) * hs + d] = o;
        }
    }
    if (P.n_splits == 1) return;
    if (tid < kv_mul) {
        const int head = kvh * kv_mul + tid;
        P.part_ml[((size_t)head * P.n_splits + split) * 2] = ml_s[2 * tid];
        P.part_ml[((size_t)head * P.n_splits + split) * 2 + 1] = ml_s[2 * tid + 1];
    }
    __threadfence();
    att_sync(bar_id);
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&P.counters[kvh], 1u);
        *is_last_p = (ticket == (unsigned int)P.n_splits - 1);
        if (*is_last_p) P.counters[kvh] = 0;  // ready for the next launch
    }
    att_sync(bar_id);
    if (!*is_last_p) return;
    __threadfence();
    // Merge the splits of this KV head (fixed order over splits).  The (max, sum) pairs of all splits are first
    // brought into shared memory with independent loads, then every thread merges one output element.
    float* ml_all = red_s;  // kv_mul * n_splits * 2 floats (n_splits <= 64 <= 2 * head_size fits the reduce buffer)
    {
        const float* src = P.part_ml + (size_t)kvh * kv_mul * P.n_splits * 2;
        for (int i = tid; i < kv_mul * P.n_splits * 2; i += ATT_THREADS) ml_all[i] = __ldcg(src + i);
    }
    att_sync(bar_id);
    for (int i = tid; i < kv_mul * hs; i += ATT_THREADS) {
        const int h = i / hs, d = i % hs;
        const int head = kvh * kv_mul + h;
        const float* ml = ml_all + h * P.n_splits * 2;
        float M = -INFINITY;
        for (int s = 0; s < P.n_splits; s++)
            if (ml[2 * s + 1] > 0.f) M = fmaxf(M, ml[2 * s]);
        const float* po = P.part_o + ((size_t)head * P.n_splits) * hs + d;
        float num = 0.f, den = 0.f;
#pragma unroll 8
        for (int s = 0; s < P.n_splits; s++) {
            const float l = ml[2 * s + 1];
            const float o = l > 0.f ? __ldcg(po + (size_t)s * hs) : 0.f;
            const float w = l > 0.f ? expf(ml[2 * s] - M) : 0.f;
            num = fmaf(w, o, num);
            den = fmaf(w, l, den);
        }
        P.out[(size_t)head * hs + d] = num / den;
    }
}


}  // namespace attn
