// Token sampler on the device (Sampler::sample, crates/slai/src/models/sampler.rs:33-131): temperature, softmax,
// then a draw from the whole distribution (sample_mult) or from the nucleus (sample_topp: candidates at or above
// (1 - topp) / (n - 1), stable order by descending probability, truncated where the cumulative probability
// exceeds topp).  The reference samples on the host after reading 128 KB of logits back every token; here the
// logits never leave the device and the generate loop stays a replayed graph.
//
// One block of 1024 threads (a vocabulary is 32-128 K entries: latency, not bandwidth).  Thread t owns the
// contiguous chunk [t*C, (t+1)*C) so that prefix sums and candidate order follow the index order of the
// reference's sequential loops; sums are block-tree sums, so probabilities agree with the reference's sequential
// f32 sums to a few ulps and the drawn id is the same unless the random number falls within that distance of a
// boundary of the cumulative distribution.
//
// The uniform random number is either passed by the caller (operator form) or derived on the device from a seed
// and the step counter: u = top 24 bits of splitmix64(seed + step) / 2^24.
#include "common.cuh"

namespace {

constexpr int ST = 1024;
constexpr int SORT_SMEM = 4096;  // candidates sorted in shared memory; more go through the global scratch

struct SampleParams {  // device-resident (the generate graph reads them from memory)
    float temperature, topp;
    unsigned long long seed;
};

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Block-wide exclusive scan of one value per thread (thread order); `total` gets the sum of all.
template <typename T>
__device__ __forceinline__ T block_excl_scan(T v, T* sh /* 33 entries */, T& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T up = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += up;
    }
    __syncthreads();
    if (lane == 31) sh[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        T w = sh[lane];
        T winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const T up = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += up;
        }
        sh[lane] = winc - w;  // exclusive prefix of the warp totals
        if (lane == 31) sh[32] = winc;
    }
    __syncthreads();
    total = sh[32];
    return sh[warp] + inc - v;
}

__device__ __forceinline__ float block_max(float v, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = sh[0];
    for (int w = 1; w < ST / 32; w++) m = fmaxf(m, sh[w]);
    return m;
}

// ascending bitonic sort of `n2` (a power of two) 64-bit keys
__device__ void bitonic_sort(unsigned long long* keys, int n2) {
    for (int k = 2; k <= n2; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n2; i += ST) {
                const int p = i ^ j;
                if (p > i) {
                    const unsigned long long a = keys[i], b = keys[p];
                    const bool up = (i & k) == 0;
                    if ((a > b) == up) {
                        keys[i] = b;
                        keys[p] = a;
                    }
                }
            }
            __syncthreads();
        }
}

__global__ void __launch_bounds__(ST) sample_kernel(float* logits, int n, const SampleParams* sp, const int* d_step, float host_coin,
                                                    int use_host_coin, unsigned long long* scratch, int scratch_cap, int* out) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float shf[33];
    __shared__ int shi[33];
    __shared__ int s_idx;
    __shared__ float s_val;
    __shared__ unsigned long long skeys[SORT_SMEM];
    const int tid = threadIdx.x;
    const float temperature = sp->temperature, topp = sp->topp;
    const int C = (n + ST - 1) / ST;
    const int i0 = min(n, tid * C), i1 = min(n, i0 + C);

    if (temperature == 0.0f) {  // greedy: first maximal index
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = i0; i < i1; i++)
            if (logits[i] > best) {
                best = logits[i];
                bi = i;
            }
        const float m = block_max(best, shf);
        if (tid == 0) s_idx = 0x7fffffff;
        __syncthreads();
        if (best == m && bi != 0x7fffffff) atomicMin(&s_idx, bi);
        __syncthreads();
        if (tid == 0) *out = s_idx == 0x7fffffff ? 0 : s_idx;
        return;
    }
    float coin = host_coin;
    if (!use_host_coin) {
        const unsigned long long h = mix64(sp->seed + (unsigned long long)(d_step ? *d_step : 0));
        coin = (float)((h >> 40) & 0xFFFFFFull) * (1.0f / 16777216.0f);
    }
    // probabilities (written over the logits, as the reference does)
    float mx = -INFINITY;
    for (int i = i0; i < i1; i++) {
        const float x = logits[i] / temperature;
        logits[i] = x;
        mx = fmaxf(mx, x);
    }
    mx = block_max(mx, shf);
    float local = 0.f;
    for (int i = i0; i < i1; i++) {
        const float e = expf(logits[i] - mx);
        logits[i] = e;
        local += e;
    }
    float sum;
    block_excl_scan(local, shf, sum);
    local = 0.f;
    for (int i = i0; i < i1; i++) {
        const float p = logits[i] / sum;
        logits[i] = p;
        local += p;
    }
    if (tid == 0) s_idx = 0x7fffffff;
    if (topp <= 0.0f || topp >= 1.0f) {  // sample_mult: first index whose inclusive prefix exceeds the coin
        float total;
        float cdf = block_excl_scan(local, shf, total);
        for (int i = i0; i < i1; i++) {
            cdf += logits[i];
            if (coin < cdf) {
                atomicMin(&s_idx, i);
                break;
            }
        }
        __syncthreads();
        if (tid == 0) *out = s_idx == 0x7fffffff ? n - 1 : s_idx;
        return;
    }
    // sample_topp: candidates in index order -> keys (descending probability, ascending index)
    const float cutoff = (1.0f - topp) / ((float)n - 1.0f);
    int cnt = 0;
    for (int i = i0; i < i1; i++) cnt += logits[i] >= cutoff;
    int n0;
    int off = block_excl_scan(cnt, shi, n0);
    if (n0 == 0) {
        // No probability reaches the cutoff (top-p below 1/n on a flat distribution, or non-finite logits).  The
        // reference underflows `n0 - 1` and panics there (models/sampler.rs:98-113); defined here as the greedy choice
        // over the probabilities: first maximal index, 0 if nothing compares.
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = i0; i < i1; i++)
            if (logits[i] > best) {
                best = logits[i];
                bi = i;
            }
        const float m = block_max(best, shf);
        if (best == m && bi != 0x7fffffff) atomicMin(&s_idx, bi);
        __syncthreads();
        if (tid == 0) *out = s_idx == 0x7fffffff ? 0 : s_idx;
        return;
    }
    const bool in_smem = n0 <= SORT_SMEM;
    int n2 = 1;
    while (n2 < n0) n2 <<= 1;
    if (!in_smem && n2 > scratch_cap) {  // cannot happen with the scratch the host sizes (next power of two of n)
        if (tid == 0) *out = 0;
        return;
    }
    unsigned long long* keys = in_smem ? skeys : scratch;
    for (int i = i0; i < i1; i++)
        if (logits[i] >= cutoff) keys[off++] = ((unsigned long long)(~__float_as_uint(logits[i])) << 32) | (unsigned int)i;
    for (int i = n0 + tid; i < n2; i += ST) keys[i] = ~0ull;
    __syncthreads();
    bitonic_sort(keys, n2);
    // cumulative probability in sorted order; truncate where it first exceeds topp
    const int C2 = (n0 + ST - 1) / ST;
    const int j0 = min(n0, tid * C2), j1 = min(n0, j0 + C2);
    float part = 0.f;
    for (int j = j0; j < j1; j++) part += __uint_as_float(~(unsigned int)(keys[j] >> 32));
    float total;
    const float base = block_excl_scan(part, shf, total);
    float cdf = base;
    for (int j = j0; j < j1; j++) {
        cdf += __uint_as_float(~(unsigned int)(keys[j] >> 32));
        if (cdf > topp) {
            atomicMin(&s_idx, j);
            break;
        }
    }
    __syncthreads();
    const int last = s_idx == 0x7fffffff ? n0 - 1 : s_idx;
    __syncthreads();
    if (last >= j0 && last < j1) {  // the owner of `last` publishes the cumulative probability up to it
        float c = base;
        for (int j = j0; j <= last; j++) c += __uint_as_float(~(unsigned int)(keys[j] >> 32));
        s_val = c;
    }
    if (tid == 0) s_idx = 0x7fffffff;
    __syncthreads();
    const float r = coin * s_val;
    cdf = base;
    for (int j = j0; j < j1 && j <= last; j++) {
        cdf += __uint_as_float(~(unsigned int)(keys[j] >> 32));
        if (r < cdf) {
            atomicMin(&s_idx, j);
            break;
        }
    }
    __syncthreads();
    if (tid == 0) {
        const int j = s_idx == 0x7fffffff ? last : s_idx;
        *out = (int)(unsigned int)(keys[j] & 0xFFFFFFFFull);
    }
}

int next_pow2(int n) {
    int p = 1;
    while (p < n) p <<= 1;
    return p;
}

}  // namespace

size_t sampler_params_bytes() { return sizeof(SampleParams); }
size_t sampler_scratch_bytes(int n) { return (size_t)next_pow2(n) * 8; }

int sampler_set_params(slai_ctx* ctx, void* d_params, float temperature, float topp, unsigned long long seed) {
    SampleParams h{temperature, topp, seed};
    SLAI_CHECK_CUDA(ctx, cudaMemcpyAsync(d_params, &h, sizeof(h), cudaMemcpyHostToDevice, ctx->stream));
    SLAI_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // `h` is a stack temporary
    return SLAI_OK;
}

int launch_sample(slai_ctx* ctx, float* d_logits, int n, const void* d_params, const int* d_step, float host_coin, bool use_host_coin,
                  void* d_scratch, int32_t* d_out, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(ST);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    SLAI_CHECK_CUDA(ctx, cudaLaunchKernelEx(&cfg, sample_kernel, d_logits, n, reinterpret_cast<const SampleParams*>(d_params), d_step, host_coin,
                                            use_host_coin ? 1 : 0, reinterpret_cast<unsigned long long*>(d_scratch), next_pow2(n), (int*)d_out));
    return SLAI_OK;
}

int ensure_scratch(slai_ctx* ctx, size_t bytes);

SLAI_API int slai_sample(slai_ctx* ctx, float* d_logits, int64_t n, float temperature, float topp, float coin, int32_t* d_token_out) {
    if (!ctx || !d_logits || !d_token_out) return SLAI_ERR_INVALID_ARG;
    SLAI_ENTER(ctx);
    SLAI_REQUIRE(ctx, n >= 2 && n <= (1 << 20), SLAI_ERR_SHAPE, "sample: vocabulary of %lld entries", (long long)n);
    SLAI_REQUIRE(ctx, temperature >= 0.0f && coin >= 0.0f && coin < 1.0f, SLAI_ERR_INVALID_ARG, "sample: temperature must be >= 0 and coin in [0, 1)");
    const size_t need = sampler_scratch_bytes((int)n) + 256;
    int rc = ensure_scratch(ctx, need);
    if (rc) return rc;
    void* d_params = reinterpret_cast<char*>(ctx->d_scratch) + sampler_scratch_bytes((int)n);
    if ((rc = sampler_set_params(ctx, d_params, temperature, topp, 0))) return rc;
    return launch_sample(ctx, d_logits, (int)n, d_params, nullptr, coin, true, ctx->d_scratch, d_token_out, false);
}
