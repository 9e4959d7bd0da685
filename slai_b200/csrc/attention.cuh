// Single-query attention over the KV cache, device side (see attention.cu for the operator and the launches).
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
    int n_heads, kv_mul, hs;  // kv_mul: query heads one work item serves (those of its virtual head)
    int kv_share = 1;         // virtual heads per cache head: virtual head v reads the keys and values of cache head v / kv_share
    const int* d_pos;
    int early = 0;  // the position scalar is final before this kernel's blocks can start (AttnLaunch::pos_stable): read it before the wait
    int n_splits;   // most splits a KV head is cut into (stride of the partial buffers)
    int tile_pos;   // positions staged in shared memory at a time
    int vec16;      // rows can be copied in 16-byte pieces (alignment of bases, strides and row length)
    float* out;
    float* part_o;   // [n_heads][n_splits][hs]
    float* part_ml;  // [n_heads][n_splits][2]
    unsigned int* counters;  // [n_kv_heads]
    PrefetchPlan ahead;      // weights of a later kernel, pulled into L2 by all blocks at the start
    // batch of query tokens (blockIdx.z): per-token strides of q / out / partials / tickets; position of token b = pos0 + b
    int batch = 0, pos0 = 0;
    long long q_bs = 0, out_bs = 0, po_bs = 0, pml_bs = 0;
    // a batch of sequences instead: token b has its own caches, cache_bs bytes after token b - 1's, and position seq_pos[b]
    long long cache_bs = 0;
    const int* seq_pos = nullptr;
#ifdef SLAI_TRACE
    unsigned long long* tl = nullptr;  // trace build only: the context's launch timeline
#endif
};

// Barrier over the ATT_THREADS threads that work on one item (named barrier `id`; id 0 with a 128-thread block is
// the block-wide barrier).
__device__ __forceinline__ void att_sync(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(ATT_THREADS) : "memory"); }

// Shared memory of one item, in bytes: q | scores | running (max, sum, rescale) | flag | one tile buffer that holds
// the K rows (padded by 16 bytes: the four threads of a position and the eight positions of a warp then hit 32
// different banks) and, once the scores are done, the V rows.  The merge of the splits reuses the tile buffer for
// the (max, sum) pairs of all splits, their weights and the partial sums of the merge's thread groups.
__host__ __device__ inline size_t attn_k_stride(int hs, int esz) { return (size_t)hs * esz + 16; }
__host__ __device__ inline size_t attn_head_bytes(int kv_mul, int hs, int tile_pos) {
    return (((size_t)kv_mul * hs + (size_t)kv_mul * tile_pos + 4 * (size_t)kv_mul + 4) * 4 + 15) & ~(size_t)15;
}
__host__ __device__ inline size_t attn_item_bytes(int kv_mul, int hs, int esz, int tile_pos, int n_splits) {
    size_t tile = tile_pos * attn_k_stride(hs, esz);
    const size_t merge = (size_t)kv_mul * n_splits * 4 * 4 + 4 * ATT_THREADS * 4;  // (max, sum) pairs of all splits, their weights, the groups' sums of the merge
    if (merge > tile) tile = merge;
    return attn_head_bytes(kv_mul, hs, tile_pos) + ((tile + 15) & ~(size_t)15);
}
// Grouped-query models would leave most SMs idle with one work item per (cache head, split): the query heads of a cache
// head are therefore dealt to `attn_kv_share(kv_mul)` virtual heads of at most two query heads each, which read the same
// keys and values (from L2 after the first).
__host__ __device__ inline int attn_kv_share(int kv_mul) { return kv_mul <= 2 ? 1 : (kv_mul % 2 == 0 ? kv_mul / 2 : kv_mul); }
// Positions per tile: at most 8 KB of K (and of V) per item -- four 16-byte pieces per thread and matrix -- a
// multiple of 8, at most 32.
__host__ __device__ inline int attn_tile_pos(int hs, int esz) {
    int t = (8192 / (hs * esz)) & ~7;
    return t < 8 ? 8 : t > 32 ? 32 : t;
}
// Splits actually used at `n` positions: one per tile, up to the maximum.
__device__ __forceinline__ int attn_splits(const AttnParams& P, int n) {
    const int want = (n + P.tile_pos - 1) / P.tile_pos;
    return want < 1 ? 1 : want > P.n_splits ? P.n_splits : want;
}

template <typename T> struct Elem;
template <> struct Elem<__half> {
    __device__ static __forceinline__ float2 ld2(const unsigned char* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
    __device__ static __forceinline__ float ld1(const unsigned char* p) { return __half2float(*reinterpret_cast<const __half*>(p)); }
};
template <> struct Elem<float> {
    __device__ static __forceinline__ float2 ld2(const unsigned char* p) { return *reinterpret_cast<const float2*>(p); }
    __device__ static __forceinline__ float ld1(const unsigned char* p) { return *reinterpret_cast<const float*>(p); }
};

// Rows of a tile travel as pieces of type V (16 bytes, or 4 when something is not 16-byte aligned); thread `tid`
// owns pieces tid, tid + 128, ...  A batch is NB pieces per thread: all its loads are issued before anything waits
// for them, so a tile costs one trip to memory.  L2 loads (ld.global.cg): the newest row was written by the kernel
// launched just before this one, on other SMs.
struct Pieces {  // (row, column) of this thread's four 16-byte pieces; the same for every tile of an item
    int r[4], c[4];
    __device__ __forceinline__ void init(int ppr, int tid) {
        int rr = tid / ppr, cc = tid - rr * ppr;
        const int dr = ATT_THREADS / ppr, dc = ATT_THREADS - dr * ppr;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            r[u] = rr;
            c[u] = cc;
            rr += dr;
            cc += dc;
            if (cc >= ppr) {
                cc -= ppr;
                rr++;
            }
        }
    }
};
__device__ __forceinline__ void load_pieces(uint4 (&buf)[4], const Pieces& w, const unsigned char* g, size_t row_pitch, int rows) {
#pragma unroll
    for (int u = 0; u < 4; u++)
        if (w.r[u] < rows) buf[u] = __ldcg(reinterpret_cast<const uint4*>(g + (size_t)w.r[u] * row_pitch) + w.c[u]);
}
__device__ __forceinline__ void store_pieces(const uint4 (&buf)[4], const Pieces& w, unsigned char* s, int row_stride, int rows) {
#pragma unroll
    for (int u = 0; u < 4; u++)
        if (w.r[u] < rows) reinterpret_cast<uint4*>(s + (size_t)w.r[u] * row_stride)[w.c[u]] = buf[u];
}
// Slow path (something is not 16-byte aligned): 4-byte pieces, one at a time.
__device__ __forceinline__ void copy_rows_u32(const unsigned char* g, size_t row_pitch, int row_bytes, int rows, unsigned char* s,
                                              int row_stride, int tid) {
    const int ppr = row_bytes >> 2, total = rows * ppr;
#pragma unroll 1
    for (int idx = tid; idx < total; idx += ATT_THREADS) {
        const int r = idx / ppr, c = idx - r * ppr;
        reinterpret_cast<unsigned int*>(s + (size_t)r * row_stride)[c] = __ldcg(reinterpret_cast<const unsigned int*>(g + (size_t)r * row_pitch) + c);
    }
}

// One work item = (virtual KV head, split `split` of `ns`) at `n` positions, processed by ATT_THREADS threads with thread
// index `tid`, shared memory `smb` (attn_item_bytes) and barrier `bar_id`.  The split's positions are walked in
// tiles with a running (max, sum) per query head (the usual streaming softmax); the partial output of the split is
// the un-normalised weighted sum of V relative to the final max.
template <typename T, int MAXQ>
__device__ __forceinline__ void attn_item(const AttnParams& P, int kvh, int split, int ns, int n, int tid, unsigned char* smb, int bar_id) {
    constexpr int ESZ = (int)sizeof(T);
    const int hs = P.hs, kv_mul = P.kv_mul, TP = P.tile_pos;
    float* q_s = reinterpret_cast<float*>(smb);       // [kv_mul][hs]
    float* sc_s = q_s + kv_mul * hs;                   // [kv_mul][TP]
    float* st_s = sc_s + kv_mul * TP;                  // [kv_mul][4]: running max, running sum, rescale of this tile
    int* is_last_p = reinterpret_cast<int*>(st_s + 4 * kv_mul);
    unsigned char* k_s = smb + attn_head_bytes(kv_mul, hs, TP);
    const int k_stride = (int)attn_k_stride(hs, ESZ);
    const int row_bytes = hs * ESZ;
    const int lane = tid & 31, warp = tid >> 5;

    const int chunk = (n + ns - 1) / ns;
    const int t0 = split * chunk;
    const int t1 = min(n, t0 + chunk);

    const int cache_head = P.kv_share > 1 ? kvh / P.kv_share : kvh;
    const unsigned char* kbase = reinterpret_cast<const unsigned char*>(P.kc) + ((size_t)cache_head * P.head_stride) * ESZ;
    const unsigned char* vbase = reinterpret_cast<const unsigned char*>(P.vc) + ((size_t)cache_head * P.head_stride) * ESZ;
    const size_t row_pitch = (size_t)P.pos_stride * ESZ;
    const float sqrt_hs = sqrtf((float)hs);
    // q: loads first, stores after the first tile's loads are in flight
    float qr[2 * MAXQ];
#pragma unroll
    for (int u = 0; u < 2 * MAXQ; u++) {
        const int i = tid + u * ATT_THREADS;
        qr[u] = i < kv_mul * hs ? __ldcg(P.q + (size_t)kvh * kv_mul * hs + i) : 0.f;
    }
    if (tid < kv_mul) {
        st_s[4 * tid] = -INFINITY;
        st_s[4 * tid + 1] = 0.f;
        st_s[4 * tid + 2] = 0.f;
    }
    float acc[MAXQ][2];
#pragma unroll
    for (int h = 0; h < MAXQ; h++) acc[h][0] = acc[h][1] = 0.f;
    Pieces pw;
    pw.init(row_bytes >> 4, tid);

    // K goes to the tile buffer; V is requested in the same trip and waits in registers until K is done with.  The pieces of
    // the next tile are requested as soon as this tile's V has left the registers, so that their trip to memory runs behind
    // the softmax and the weighted sum.
    uint4 kb[4], vb[4];
    if (P.vec16 && t0 < t1) {
        const int cnt0 = min(TP, t1 - t0);
        load_pieces(kb, pw, kbase + (size_t)t0 * row_pitch, row_pitch, cnt0);
        load_pieces(vb, pw, vbase + (size_t)t0 * row_pitch, row_pitch, cnt0);
    }
#pragma unroll 1
    for (int tt = t0; tt < t1; tt += TP) {
        const int cnt = min(TP, t1 - tt);
        if (tt != t0) att_sync(bar_id);  // the previous tile has been consumed
        if (P.vec16) store_pieces(kb, pw, k_s, k_stride, cnt);
        else copy_rows_u32(kbase + (size_t)tt * row_pitch, row_pitch, row_bytes, cnt, k_s, k_stride, tid);
        if (tt == t0) {
#pragma unroll
            for (int u = 0; u < 2 * MAXQ; u++) {
                const int i = tid + u * ATT_THREADS;
                if (i < kv_mul * hs) q_s[i] = qr[u];
            }
        }
        att_sync(bar_id);
        // scores: four threads per position, 32 positions per pass
        {
            const int c = tid & 3;
#pragma unroll 1
#pragma unroll 1
            for (int i0 = 0; i0 < cnt; i0 += 32) {
                const int i = i0 + (tid >> 2);
                float part[MAXQ];
#pragma unroll
                for (int h = 0; h < MAXQ; h++) part[h] = 0.f;
                if (i < cnt) {
                    const unsigned char* kp = k_s + (size_t)i * k_stride;
#pragma unroll 4
#pragma unroll 4
                    for (int e = c; e < (hs >> 1); e += 4) {
                        const float2 k2 = Elem<T>::ld2(kp + 2 * e * ESZ);
#pragma unroll
                        for (int h = 0; h < MAXQ; h++)
                            if (h < kv_mul) part[h] = fmaf(k2.y, q_s[h * hs + 2 * e + 1], fmaf(k2.x, q_s[h * hs + 2 * e], part[h]));
                    }
                }
#pragma unroll
                for (int h = 0; h < MAXQ; h++) {
                    part[h] += __shfl_xor_sync(0xffffffffu, part[h], 1);
                    part[h] += __shfl_xor_sync(0xffffffffu, part[h], 2);
                }
                if (i < cnt && c == 0) {
#pragma unroll
                    for (int h = 0; h < MAXQ; h++)
                        if (h < kv_mul) sc_s[h * TP + i] = part[h] / sqrt_hs;
                }
            }
        }
        att_sync(bar_id);
        // the K rows are done with: V takes their place (read by the last step of this tile)
        if (P.vec16) {
            store_pieces(vb, pw, k_s, row_bytes, cnt);
            if (tt + TP < t1) {
                const int cn = min(TP, t1 - (tt + TP));
                load_pieces(kb, pw, kbase + (size_t)(tt + TP) * row_pitch, row_pitch, cn);
                load_pieces(vb, pw, vbase + (size_t)(tt + TP) * row_pitch, row_pitch, cn);
            }
        } else {
            copy_rows_u32(vbase + (size_t)tt * row_pitch, row_pitch, row_bytes, cnt, k_s, row_bytes, tid);
        }
        // running softmax per query head
#pragma unroll 1
        for (int h = warp; h < kv_mul; h += ATT_WARPS) {
            const float m_old = st_s[4 * h], l_old = st_s[4 * h + 1];
            float m = m_old;
#pragma unroll 1
            for (int i = lane; i < cnt; i += 32) m = fmaxf(m, sc_s[h * TP + i]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            float l = 0.f;
#pragma unroll 1
            for (int i = lane; i < cnt; i += 32) {
                const float p = expf(sc_s[h * TP + i] - m);
                sc_s[h * TP + i] = p;
                l += p;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            __syncwarp();
            if (lane == 0) {
                const float resc = m_old == -INFINITY ? 0.f : expf(m_old - m);
                st_s[4 * h] = m;
                st_s[4 * h + 1] = l_old * resc + l;
                st_s[4 * h + 2] = resc;
            }
        }
        att_sync(bar_id);
        // weighted sum of V: thread `tid` owns dims tid and tid + 128
#pragma unroll
        for (int jj = 0; jj < 2; jj++) {
            const int d = tid + jj * ATT_THREADS;
            if (d < hs) {
                float a[MAXQ];
#pragma unroll
                for (int h = 0; h < MAXQ; h++) a[h] = h < kv_mul ? acc[h][jj] * st_s[4 * h + 2] : 0.f;
#pragma unroll 4
#pragma unroll 4
                for (int i = 0; i < cnt; i++) {
                    const float v = Elem<T>::ld1(k_s + (size_t)i * row_bytes + (size_t)d * ESZ);
#pragma unroll
                    for (int h = 0; h < MAXQ; h++)
                        if (h < kv_mul) a[h] = fmaf(sc_s[h * TP + i], v, a[h]);
                }
#pragma unroll
                for (int h = 0; h < MAXQ; h++) acc[h][jj] = a[h];
            }
        }
    }
    // partial (or final) output
#pragma unroll
    for (int jj = 0; jj < 2; jj++) {
        const int d = tid + jj * ATT_THREADS;
        if (d < hs) {
#pragma unroll
            for (int h = 0; h < MAXQ; h++)
                if (h < kv_mul) {
                    const int head = kvh * kv_mul + h;
                    if (ns == 1) P.out[(size_t)head * hs + d] = acc[h][jj] / st_s[4 * h + 1];
                    else P.part_o[((size_t)head * P.n_splits + split) * hs + d] = acc[h][jj];
                }
        }
    }
    if (ns == 1) return;
    if (tid < kv_mul) {
        const int head = kvh * kv_mul + tid;
        P.part_ml[((size_t)head * P.n_splits + split) * 2] = st_s[4 * tid];
        P.part_ml[((size_t)head * P.n_splits + split) * 2 + 1] = st_s[4 * tid + 1];
    }
    att_sync(bar_id);
    if (tid == 0) {
        __threadfence();  // cumulative: orders the whole block's partials (seen through the barrier) before the ticket
        const unsigned int ticket = atomicAdd(&P.counters[kvh], 1u);
        *is_last_p = (ticket == (unsigned int)ns - 1);
        if (*is_last_p) P.counters[kvh] = 0;  // ready for the next launch
    }
    att_sync(bar_id);
    if (!*is_last_p) return;
    __threadfence();
    // Merge the splits of this KV head (fixed order over splits).  The (max, sum) pairs of all splits come into
    // shared memory with independent loads and are turned into weights once; every thread then combines its
    // output elements, sixteen independent loads at a time.
    float* ml_all = reinterpret_cast<float*>(k_s);  // [kv_mul][ns][2] (max, sum), then [kv_mul][ns][2] (weight, weight*sum)
    float* w_all = ml_all + kv_mul * ns * 2;
#pragma unroll 1
    for (int i = tid; i < kv_mul * ns * 2; i += ATT_THREADS) {
        const int h = i / (2 * ns), r = i - h * 2 * ns;
        ml_all[i] = __ldcg(P.part_ml + ((size_t)(kvh * kv_mul + h) * P.n_splits) * 2 + r);
    }
    att_sync(bar_id);
#pragma unroll 1
    for (int i = tid; i < kv_mul * ns; i += ATT_THREADS) {
        const int h = i / ns;
        const float* ml = ml_all + h * ns * 2;
        float M = -INFINITY;
#pragma unroll 1
        for (int s = 0; s < ns; s++)
            if (ml[2 * s + 1] > 0.f) M = fmaxf(M, ml[2 * s]);
        const float l = ml_all[2 * i + 1];
        const float w = l > 0.f ? expf(ml_all[2 * i] - M) : 0.f;
        w_all[2 * i] = w;
        w_all[2 * i + 1] = w * l;
    }
    att_sync(bar_id);
    if (ns > 32 && (hs & 3) == 0 && (hs >> 2) <= ATT_THREADS / 2) {
        // Many splits (measured: pays from three rounds of sixteen loads on; with fewer the plain loop below is quicker).
        // Threads as (group g, 16-byte chunk c of the head's output): group g adds the splits s = g, g + G, ... of its chunk
        // (all of a thread's loads are independent: one trip to memory for up to 16 splits per group), the groups' sums
        // meet in shared memory and are added in group order.  Fixed order throughout.
        const int chunks = hs >> 2, G = ATT_THREADS / chunks;
        const int c = tid % chunks, g = tid / chunks;
        float* gsum = w_all + kv_mul * ns * 2;  // [G][hs]
#pragma unroll 1
        for (int h = 0; h < kv_mul; h++) {
            const int head = kvh * kv_mul + h;
            const float* wl = w_all + h * ns * 2;
            float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g < G) {
                const float4* po = reinterpret_cast<const float4*>(P.part_o + ((size_t)head * P.n_splits) * hs) + c;
#pragma unroll 1
                for (int s0 = g; s0 < ns; s0 += 16 * G) {
                    float4 o[16];
#pragma unroll
                    for (int u = 0; u < 16; u++) o[u] = s0 + u * G < ns ? __ldcg(po + (size_t)(s0 + u * G) * chunks) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 16; u++)
                        if (s0 + u * G < ns) {
                            const float w = wl[2 * (s0 + u * G)];
                            if (w > 0.f) {
                                num.x = fmaf(w, o[u].x, num.x); num.y = fmaf(w, o[u].y, num.y);
                                num.z = fmaf(w, o[u].z, num.z); num.w = fmaf(w, o[u].w, num.w);
                            }
                        }
                }
                *reinterpret_cast<float4*>(gsum + g * hs + 4 * c) = num;
            }
            att_sync(bar_id);
            if (tid < hs) {
                float nsum = 0.f, den = 0.f;
                for (int gg = 0; gg < G; gg++) nsum += gsum[gg * hs + tid];
                for (int sp = 0; sp < ns; sp++) den += wl[2 * sp + 1];
                P.out[(size_t)head * hs + tid] = nsum / den;
            }
            att_sync(bar_id);  // gsum is reused by the next head
        }
        return;
    }
#pragma unroll 1
    for (int i = tid; i < kv_mul * hs; i += ATT_THREADS) {
        const int h = i / hs, d = i - h * hs;
        const int head = kvh * kv_mul + h;
        const float* wl = w_all + h * ns * 2;
        const float* po = P.part_o + ((size_t)head * P.n_splits) * hs + d;
        float num = 0.f, den = 0.f;
#pragma unroll 1
        for (int s0 = 0; s0 < ns; s0 += 16) {
            float o[16];
#pragma unroll
            for (int u = 0; u < 16; u++) o[u] = s0 + u < ns ? __ldcg(po + (size_t)(s0 + u) * hs) : 0.f;
#pragma unroll
            for (int u = 0; u < 16; u++)
                if (s0 + u < ns) {
                    const float w = wl[2 * (s0 + u)];
                    num = fmaf(w, w > 0.f ? o[u] : 0.f, num);
                    den += wl[2 * (s0 + u) + 1];
                }
        }
        P.out[(size_t)head * hs + d] = num / den;
    }
}

}  // namespace attn
