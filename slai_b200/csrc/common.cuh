// Shared declarations of the slai_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <atomic>
#include <string>
#include <vector>
#include <unordered_map>

#include "../../include/slai_b200.h"

#define SLAI_API extern "C" __attribute__((visibility("default")))

struct RopeTable {
    int head_size;
    float base;
    float* d_theta;  // head_size/2 inverse frequencies, computed on the host with libm powf
};

// Tensor-parallel exchange over peer memory (tp.cu): every rank owns a region [2 parities][ranks][XCHG_MAX_DIM] of
// (value, sequence tag) pairs; peers store their partial vectors straight into it over NVLink, one 8-byte store per
// element, and the reader knows an element has arrived when its tag equals the exchange's sequence number.
constexpr int XCHG_MAX_RANKS = 8;
constexpr int XCHG_MAX_DIM = 16384;
struct PeerExchange {
    int ranks, rank;
    uint2* slot_at[XCHG_MAX_RANKS];  // base of every rank's region (own region included), as seen from here
    uint2* local_sum;                // [2 parities][XCHG_MAX_DIM]: this GPU's two-level sums (never written by peers)
    unsigned int* d_tokseq;          // device scalar (local): tokens decoded so far (one tick per token)
};

struct slai_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    std::string last_error;
    bool use_pdl = true;            // programmatic dependent launch between decode kernels
    void* d_scratch = nullptr;      // attention split partials etc.
    size_t scratch_bytes = 0;
    std::vector<void*> retired_scratch;  // outgrown scratch buffers: recorded passes may still point at them, freed with the context
    std::vector<RopeTable> rope_tables;
    unsigned long long* trace_buf = nullptr;  // trace build only: per-block stamps of the last 64 GEMV launches
    unsigned long long trace_launches = 0;
    unsigned long long* tl = nullptr;         // trace build only: the launch timeline
    unsigned int* d_counters = nullptr;  // CNT_WORDS zeroed words, see the map below
    unsigned int wait_limit = 1u << 20;  // rounds a bounded device-side wait polls before it gives up (slai_ctx_set_wait_limit)
    // tensor-parallel group (tp.cu): NCCL communicator of this context's rank, null when not sharded
    void* tp_comm = nullptr;
    int tp_rank = 0, tp_size = 1;
    PeerExchange xchg = {};     // filled by slai_tp_peer_attach
    void* xchg_region = nullptr;  // this rank's region (device memory, exported to the peers)
    bool xchg_ready = false;
    bool xchg_loopback = false;   // slai_tp_peer_loopback: the region stands in for every rank's (single-GPU testing)
    // slai_llama_stats: while `stats_on`, the GEMV and attention launchers bracket their kernels with events
    bool stats_on = false;
    std::vector<cudaEvent_t> stats_ev;
    std::vector<int> stats_cls;   // class of the interval that ends at the event of the same index (STATS_* below)
};
// Kernel classes of slai_llama_stats (index into slai_llama_stats_t::us).
enum { STATS_OTHER = 0, STATS_QKV = 1, STATS_ATTENTION = 2, STATS_WO = 3, STATS_GATE_UP = 4, STATS_DOWN = 5, STATS_LOGITS = 6, STATS_CLASSES = 7 };
// Ends an interval of class `cls` on the context's stream (no-op unless statistics are being taken).
int slai_stats_mark(slai_ctx* ctx, int cls);

// tp.cu: sum of `n` floats over the ranks of the context's group, on the context's stream
int tp_all_reduce_sum(slai_ctx* ctx, const float* d_in, float* d_out, int64_t n);
// tp.cu: concatenation in rank order of every rank's `n` floats, on the context's stream
int tp_all_gather(slai_ctx* ctx, const float* d_in, float* d_out, int64_t n);
// tp.cu: one more token decoded (sequence numbers of the peer exchange derive from it)
int tp_tick(slai_ctx* ctx);

// Map of slai_ctx::d_counters (unsigned words, all zero between launches).
constexpr int CNT_ATTN_TICKETS = 0;    // one ticket per KV head (<= 1024): last split of a head merges the partials
constexpr int CNT_ARGMAX = 1100;       // ticket, then per-block (value, index) pairs of the multi-block argmax
constexpr int CNT_ATTN_POS = 2048;     // position scalar of the stand-alone slai_attention
constexpr int CNT_ERR_FLAG = 3000;     // raised by a bounded wait that ran out (1 weight ring, 2 grid barrier, 3 peer exchange)
constexpr int CNT_WORDS = 4096;

int slai_set_error(slai_ctx* ctx, int code, const char* fmt, ...);
int slai_check_wait_flag(slai_ctx* ctx);  // ops.cu: SLAI_ERR_TIMEOUT if a bounded device-side wait ran out (stream must be idle)

// Every exported function runs with its context's device current and puts the caller's device back on return, so
// several contexts (one per GPU) can be driven from one thread.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};
#define SLAI_ENTER(ctx) DeviceGuard slai_device_guard_((ctx)->device)

// Kernel attributes (the dynamic shared-memory opt-in) are per device: one flag per device and kernel instantiation.
constexpr int SLAI_MAX_DEVICES = 64;
struct PerDeviceOnce {
    std::atomic<bool> done[SLAI_MAX_DEVICES];
    bool need(int dev) const { return dev < 0 || dev >= SLAI_MAX_DEVICES || !done[dev].load(std::memory_order_acquire); }
    void set(int dev) {
        if (dev >= 0 && dev < SLAI_MAX_DEVICES) done[dev].store(true, std::memory_order_release);
    }
};

#define SLAI_CHECK_CUDA(ctx, expr)                                                                 \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return slai_set_error((ctx), SLAI_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,            \
                                  cudaGetErrorString(_e), __FILE__, __LINE__);                     \
    } while (0)

#define SLAI_REQUIRE(ctx, cond, code, ...)                                                         \
    do {                                                                                           \
        if (!(cond)) return slai_set_error((ctx), (code), __VA_ARGS__);                            \
    } while (0)

// ------------------------------------------------------------------------------------------------
// Weights that a LATER kernel of the decode step will stream, pulled into L2 by the blocks of the current kernel as
// soon as they start.  A decode kernel spends microseconds in phases that move no weight bytes (waiting for its
// predecessor, staging its input vector, the epilogue); with the next kernel's weights requested one kernel ahead
// the HBM stream runs through those phases and the next kernel's ring fills from L2.  Off unless SLAI_AHEAD_MB is set:
// the main loop consumes no faster from L2 than from HBM, and the requests lengthen the hand-over (measured).
// ------------------------------------------------------------------------------------------------
struct PrefetchPlan {
    const char* ptr[3] = {nullptr, nullptr, nullptr};  // 16-byte aligned
    unsigned long long bytes[3] = {0, 0, 0};
};
#ifdef __CUDACC__
// Chunk c of a range goes to block c % nblocks, thread c / nblocks: every block issues a few requests, spread over
// the whole range.  The requests are fire-and-forget (no completion is awaited, nothing lands in the SM).
__device__ __forceinline__ void prefetch_plan_issue(const PrefetchPlan& pf, int block, int nblocks, int tid, int nthreads) {
    constexpr unsigned long long CH = 8192;
#pragma unroll
    for (int r = 0; r < 3; r++) {
        const unsigned long long n = pf.bytes[r];
        if (n == 0) continue;
        const long long nch = (long long)((n + CH - 1) / CH);
        for (long long c = block + (long long)nblocks * tid; c < nch; c += (long long)nblocks * nthreads) {
            const unsigned long long off = (unsigned long long)c * CH;
            const unsigned int len = (unsigned int)((n - off < CH ? n - off : CH) & ~15ull);
            if (len) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf.ptr[r] + off), "r"(len) : "memory");
        }
    }
}
#endif

// ------------------------------------------------------------------------------------------------
// Quantized matrix as stored on the device: tile-major blocks of 16 rows x one K step (layout.cuh);
// F32 matrices are dense row-major.  The last tile is padded with zero rows.
// ------------------------------------------------------------------------------------------------
struct slai_qmatrix {
    slai_ctx* ctx = nullptr;
    int fmt = 0;      // format of the device data (what the kernels see)
    int src_fmt = 0;  // format of the blocks the caller uploaded (differs for the legacy formats, see legacy_device_format)
    int64_t nrows = 0, ncols = 0;
    int64_t tile_bytes = 0;  // bytes of one 16-row tile (F32: bytes of one row)
    uint8_t* data = nullptr;
    size_t bytes = 0;
    bool owns = true;
};

// The legacy 32-element formats and Q8_K have no kernels of their own.  Q4_0 and Q5_0 are re-expressed exactly as
// Q8_0 at upload (same f16 scale, quant - 8 / - 16 as int8: (q - 8) * d is the very product Q8_0 evaluates); Q4_1,
// Q5_1 (scale and offset) and Q8_K (f32 scale) are dequantised to dense f32 with the reference's rounding, which is
// what the reference itself does with tensors its quantised kernels do not take (gguf.rs:148-162).
static inline int legacy_device_format(int fmt) {
    switch (fmt) {
        case SLAI_FMT_Q4_0:
        case SLAI_FMT_Q5_0: return SLAI_FMT_Q8_0;
        case SLAI_FMT_Q4_1:
        case SLAI_FMT_Q5_1:
        case SLAI_FMT_Q8_K: return SLAI_FMT_F32;
    }
    return fmt;
}
static inline int fmt_block_elems(int fmt) {
    switch (fmt) {
        case SLAI_FMT_F32: return 1;
        case SLAI_FMT_Q4_0:
        case SLAI_FMT_Q4_1:
        case SLAI_FMT_Q5_0:
        case SLAI_FMT_Q5_1:
        case SLAI_FMT_Q8_0: return 32;
        case SLAI_FMT_Q8_K:
        case SLAI_FMT_Q4_K:
        case SLAI_FMT_Q5_K:
        case SLAI_FMT_Q6_K: return 256;
    }
    return 0;
}
static inline int fmt_block_bytes(int fmt) {
    switch (fmt) {
        case SLAI_FMT_F32: return 4;
        case SLAI_FMT_Q4_0: return 18;
        case SLAI_FMT_Q4_1: return 20;
        case SLAI_FMT_Q5_0: return 22;
        case SLAI_FMT_Q5_1: return 24;
        case SLAI_FMT_Q8_K: return 292;
        case SLAI_FMT_Q8_0: return 34;
        case SLAI_FMT_Q4_K: return 144;
        case SLAI_FMT_Q5_K: return 176;
        case SLAI_FMT_Q6_K: return 210;
    }
    return 0;
}
static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// ------------------------------------------------------------------------------------------------
// GEMV launch description (gemv.cu).  One launch covers up to three matrices that share the input
// vector (q/k/v or gate/up); the rows of all segments form one virtual row space tiled by 16.
// ------------------------------------------------------------------------------------------------
enum GemvPrologue { PRO_NONE = 0, PRO_RMS = 1, PRO_LN = 2 };
enum GemvEpilogue {
    EPI_STORE = 0,     // out[r] = acc (+bias)
    EPI_RESID = 1,     // out[r] = resid[r] + acc (+bias)       (out may alias resid)
    EPI_SILU = 2,      // segments 0/1 = gate/up: out[r] = up * gate / (1 + exp(-gate))
    EPI_GELU = 3,      // out[r] = gelu(acc + bias)
    EPI_QKV = 4,       // segments q,k,v: optional bias, optional adjacent-pair RoPE on q,k; q -> out f32,
                       // k,v -> KV cache at position *d_pos
    EPI_XCHG = 5       // tensor parallel: acc (+resid on rank 0) stored into every rank's exchange slot (PeerExchange)
};


struct GemvSeg {
    const uint8_t* w = nullptr;   // first tile of the segment (tile-major data; F32: first row)
    int64_t tile_bytes = 0;       // bytes of one 16-row tile
    int rows = 0;                 // logical rows
    int tile0 = 0;                // first 16-row tile of this segment in the virtual tile space (set by gemv_launch)
    const float* bias = nullptr;  // per row of the segment, may be null
    int out_off = 0;              // index in `out` of the segment's row 0
    int role = 0;                 // EPI_QKV: 0 = q (to `out`), 1 = k, 2 = v (to the caches)
};

struct GemvLaunch {
    int fmt = 0;
    int K = 0;
    int nseg = 1;
    GemvSeg seg[3];
    const float* v = nullptr;  // input vector (K floats)
    float* out = nullptr;
    int pro = PRO_NONE;
    const float* norm_w = nullptr;  // RMS weight or LN gamma
    const float* norm_b = nullptr;  // LN beta
    float eps = 0.f;
    int epi = EPI_STORE;
    const float* resid = nullptr;
    // EPI_QKV
    int rope = 0;                  // 1: rotate adjacent pairs of q and k
    const float* rope_theta = nullptr;  // head_size/2 inverse frequencies
    const float* rope_cs = nullptr;     // optional: (cos, sin) of this token's angles, head_size/2 pairs (else sincosf in the epilogue)
    int head_size = 0;
    const int* d_pos = nullptr;    // device scalar: position (RoPE angle and KV slot)
    void* kcache = nullptr;        // layer base of the K cache
    void* vcache = nullptr;
    float* k_out = nullptr;        // EPI_QKV: the k rows go here as f32 (kv_dim floats) instead of the cache (a rotation that
                                   // pairs rows half a head apart is applied afterwards, by rope_kv_store_launch)
    int kv_dtype = SLAI_KV_F16;
    int64_t kv_pos_stride = 0;     // elements between positions
    int64_t kv_head_stride = 0;    // elements between heads
    bool pdl = false;              // launch with programmatic stream serialization
    const void* prefetch = nullptr;  // what the next kernel reads first (e.g. its norm weights): pulled into L2 meanwhile
    size_t prefetch_bytes = 0;
    PrefetchPlan ahead;              // weights of a later kernel: pulled into L2 by this one (see PrefetchPlan)
    int stats_cls = -1;              // slai_llama_stats class of this launch (-1: derived from the epilogue)
    // tensor-parallel exchange over peer memory (null: not used)
    const PeerExchange* xchg = nullptr;
    int xchg_out_idx1 = 0;         // EPI_XCHG: index + 1 of this exchange inside the token
    int xchg_in_idx1 = 0;          // > 0: the input vector is the sum over ranks of exchange idx (instead of `v`)
    int xchg_per_token = 0;
    float* xsum_out = nullptr;     // with xchg_in: where block 0 leaves the summed vector
};

int gemv_launch(slai_ctx* ctx, const GemvLaunch& L);
// gemv_batch.cu: out[b][m] = sum_k W[m][k] v[b][k] for a batch of 2..8 vectors in one pass over a quantised matrix
bool gemv_batch_supported(const slai_qmatrix* w);
enum { BATCH_STORE = 0, BATCH_ADD = 1, BATCH_SILU = 2, BATCH_PAIR_SILU = 3 };
// the same for the concatenation by rows of up to three matrices that share the input (see gemv_batch.cu)
int gemv_batch_launch_multi(slai_ctx* ctx, float* d_out, const slai_qmatrix* const* ws, int nw, const float* d_v, int n_batch, long long ldo,
                            int epi, const float* d_gate);
int gemv_batch_launch(slai_ctx* ctx, float* d_out, const slai_qmatrix* w, const float* d_v, int n_batch, long long ldo = 0, int epi = BATCH_STORE,
                      const float* d_gate = nullptr);

// attention.cu
struct AttnLaunch {
    const float* q;
    const void* kcache;
    const void* vcache;
    int kv_dtype;
    int64_t pos_stride, head_stride;  // in elements
    int n_heads, kv_mul, head_size;
    const int* d_pos;   // device scalar position (attends to 0..=pos)
    int max_pos;        // upper bound of *d_pos (sizes the split)
    float* out;         // n_heads*head_size
    bool pdl;
    void* scratch;      // split partials; NULL = the context's scratch (grown on demand, not graph-safe)
    size_t scratch_bytes;
    PrefetchPlan ahead; // weights of a later kernel: pulled into L2 by this one
    // A batch of query tokens (prompt processing): token b reads q + b * q_batch_stride, attends to positions
    // 0..=pos0 + b, writes out + b * out_batch_stride; d_pos is ignored.  `scratch` then holds `batch` times the
    // per-token partials and `batch_counters` one zeroed ticket per (token, KV head).
    int batch = 0;
    int pos0 = 0;
    long long q_batch_stride = 0, out_batch_stride = 0;
    unsigned int* batch_counters = nullptr;
    // A batch of sequences instead (one query token of each): token b reads the caches `cache_batch_stride` bytes after token
    // b - 1's and attends to positions 0..=d_pos_batch[b] (a negative position: nothing is done for b).
    long long cache_batch_stride = 0;
    const int* d_pos_batch = nullptr;
    // *d_pos was written by a kernel that has completed before any block of this one can start, so it may be read before the
    // dependency wait.  True inside a decode step: the scalar is written once per token, and the embedding kernel that
    // follows neither starts before that write is complete nor lets its own dependents start before it has finished.
    bool pos_stable = false;
};
size_t attention_scratch_bytes(slai_ctx* ctx, int n_heads, int kv_mul, int head_size, int max_pos);
int attention_launch(slai_ctx* ctx, const AttnLaunch& A);
int attention_tickets(int n_heads, int kv_mul);  // tickets (unsigned words) one query token's launch uses
int ensure_scratch(slai_ctx* ctx, size_t bytes);
const float* rope_table(slai_ctx* ctx, int head_size, float base);

// ops.cu helpers used by the models
int launch_embed_f32(slai_ctx* ctx, float* x, const float* table, int dim, const int* d_token, const float* wpe,
                     const int* d_pos, bool pdl, const float* rope_theta = nullptr, float* rope_cs = nullptr, int rope_half = 0);
int launch_embed_q8(slai_ctx* ctx, float* x, const slai_qmatrix* wte, const int* d_token, const float* wpe,
                    const int* d_pos, bool pdl, const float* rope_theta = nullptr, float* rope_cs = nullptr, int rope_half = 0);
int launch_argmax(slai_ctx* ctx, const float* v, int64_t n, int32_t* d_out, bool pdl);
int rms_norm_rows_launch(slai_ctx* ctx, float* d_out, const float* d_x, const float* d_w, int64_t n, int rows, float eps);
// sampler.cu
size_t sampler_params_bytes();
size_t sampler_scratch_bytes(int n);
int sampler_set_params(slai_ctx* ctx, void* d_params, float temperature, float topp, unsigned long long seed);
int launch_sample(slai_ctx* ctx, float* d_logits, int n, const void* d_params, const int* d_step, float host_coin, bool use_host_coin,
                  void* d_scratch, int32_t* d_out, bool pdl);
int launch_advance(slai_ctx* ctx, int* d_token, int* d_pos, const int32_t* d_next, int32_t* d_history, int vocab, bool pdl);

// ------------------------------------------------------------------------------------------------
// Trace build (-DSLAI_TRACE, `python -m slai_b200.build --trace` -> libslai_b200_trace.so; reader: slai_b200/trace.py).
// Thread 0 of every GEMV block stamps %globaltimer at fixed points into the context's trace buffer; block 0 of every
// GEMV / attention launch appends one record {kernel id, 7 stamps} to a device-side timeline, in execution order.
// It works inside CUDA graphs, so the decode step is seen exactly as it runs.  The shipped library has none of it.
// ------------------------------------------------------------------------------------------------
#ifdef SLAI_TRACE
constexpr int TL_SLOTS = 16, TL_CAP = 4096;  // slai_ctx::tl: TL_CAP records of TL_SLOTS words, then the record counter
constexpr int TRACE_POINTS = 16, TRACE_BLOCKS = 256;  // per launch: stamps of every block (slai_ctx::trace_buf, 64 launches deep)
#endif
#if defined(SLAI_TRACE) && defined(__CUDACC__)
__device__ __forceinline__ unsigned long long slai_globaltimer() {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
    return gt;
}
// stamps[0..14] of block 0 of the launch.  GEMV: 0 start, 1 barriers initialised, 2 first weight blocks requested,
// 3 dependents released and look-ahead issued, 4 predecessor done, 5 partial sums cleared, 6 input loaded and its
// statistics summed per thread, 7 statistics reduced over the block, 8 digits written, 9 staged (barrier), 10 main
// loop done, 11 partial sums complete (barrier), 12 epilogue done, 13 end.  Attention: 0 start, 4 predecessor done, 13 end.
__device__ __forceinline__ void slai_tl_append(unsigned long long* tl, unsigned long long id, const unsigned long long* stamps) {
    const unsigned long long i = atomicAdd(tl + TL_SLOTS * TL_CAP, 1ull) % TL_CAP;
    tl[TL_SLOTS * i] = id;
    for (int k = 0; k < TL_SLOTS - 1; k++) tl[TL_SLOTS * i + 1 + k] = stamps[k];
}
#endif

// prefill.cu: prompt processing as GEMMs on the tcgen05 tensor cores
struct PrefillGemm {
    const slai_qmatrix* w = nullptr;  // quantised matrix [rows_total x K]; the first `rows` rows are used
    int rows = 0;
    const __half* x_hi = nullptr;     // activations as fp16 pairs (x = hi + lo), planes of [t_pad][K]
    const __half* x_lo = nullptr;
    int T = 0, t_pad = 0, NT = 0;     // valid tokens, allocated rows (multiple of NT), tokens per CTA tile
    float* out = nullptr;             // [T][ldo], row m of the product at column out_off + m
    int ldo = 0, out_off = 0;
    const float* resid = nullptr;     // optional [T][ldr]: out = resid + product (may alias out)
    int ldr = 0;
    const float* bias = nullptr;      // optional [rows]
};
size_t prefill_gemm_smem(int NT);
int prefill_gemm_launch(slai_ctx* ctx, const PrefillGemm& G);
int prefill_split_launch(slai_ctx* ctx, const float* x, int ldx, const float* norm_w, float eps, int T, int K, __half* hi, __half* lo);
int prefill_silu_split_launch(slai_ctx* ctx, const float* gate, const float* up, int T, int H, __half* hi, __half* lo);
int prefill_split_ln_launch(slai_ctx* ctx, const float* x, int ldx, const float* gamma, const float* beta, float eps, int T, int K, __half* hi,
                            __half* lo);
int prefill_gelu_split_launch(slai_ctx* ctx, const float* g, int T, int H, __half* hi, __half* lo);
int prefill_add_rows_launch(slai_ctx* ctx, float* x, int dim, const float* table, int pos0, int T);
int prefill_embed_launch(slai_ctx* ctx, float* x, int dim, const int* d_tokens, int T, const float* table, const slai_qmatrix* qtable);
// One token of each of `B` sequences: row b of qkv ([B][ld]: q, k, v side by side) at position d_pos[b] (negative: skipped),
// q rotated into q_out ([B][q_dim]), k and v into the caches of sequence b, `seq_stride` bytes after those of sequence b - 1.
int rope_kv_store_seqs_launch(slai_ctx* ctx, const float* qkv, int ld, int q_dim, int kv_dim, int head_size, const int* d_pos, int B,
                              const float* theta, int neox, float* q_out, void* kcache, void* vcache, int kv_f16, long long kv_head_stride,
                              long long seq_stride);
int rope_kv_store_launch(slai_ctx* ctx, float* q, const float* k, const float* v, int q_dim, int kv_dim, int head_size, const int* d_pos,
                         const float* theta, int neox, void* kcache, void* vcache, int kv_f16, long long kv_head_stride, bool pdl);
bool prefill_attention_supported(int head_size, int kv_f16, const void* kc, const void* vc, long long head_stride);
int prefill_attention_launch(slai_ctx* ctx, const float* q, int q_ld, const void* kc, const void* vc, int kv_f16, long long head_stride, int head_size,
                             int n_heads, int kv_mul, int pos0, int T, float* out, int out_ld);
int prefill_rope_kv_launch(slai_ctx* ctx, const float* qkv, int ld, int q_dim, int kv_dim, int head_size, int pos0, int T,
                           const float* theta, int neox, float* q_out, void* kcache, void* vcache, int kv_f16, long long kv_head_stride);

size_t gemv_dig_region(int fmt, int K);
