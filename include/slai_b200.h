/*
 * slai_b200 — C ABI of the B200 (sm_100a) backend for slai's per-token decode path.
 *
 * Every entry point replaces one Rust interface of dimforge/slai (cited as file:line inside that
 * project).  The reference has no C ABI: its GPU boundary is the generic `B: Backend` of the external
 * `slang-hal` crate plus the per-operator `launch` methods; a Rust shim (rust/slai-b200-sys) binds the
 * functions below so those `launch` signatures keep their shape.
 *
 * Conventions
 *  - All functions return an `int` status (SLAI_OK == 0); nothing aborts or throws across the boundary.
 *    `slai_last_error_string` gives the text of the last failure on a context.
 *  - Pointers named `d_*` are CUDA device pointers owned by the caller (allocated with `slai_malloc` or
 *    any CUDA allocator on the same device); the library neither frees nor keeps them after the call's
 *    stream work.  Pointers named `h_*` are host pointers.
 *  - Calls enqueue work on the context's stream and return ("record, then run", like a `B::Pass`);
 *    `slai_ctx_sync` and the calls documented as blocking are the only ones that wait.
 *  - A context is not thread-safe: one host thread at a time.  Contexts on different GPUs are independent.
 *  - There is no CPU fallback: without a CUDA device every call fails with SLAI_ERR_CUDA.
 */
#ifndef SLAI_B200_H
#define SLAI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct slai_ctx slai_ctx;         /* LlmOps<B> + backend + one stream (context.rs:29-96)      */
typedef struct slai_qmatrix slai_qmatrix; /* GpuQuantMatrix<B> (quantized_matrix.rs:11-22)            */
typedef struct slai_llama slai_llama;     /* Llama2State + Llama2Weights (models/llama2/transformer.rs) */
typedef struct slai_gpt2 slai_gpt2;       /* Gpt2Model (models/gpt2/cpu.rs:66-112)                    */
typedef struct slai_tp slai_tp;           /* tensor-parallel group (no counterpart in the reference)  */

enum slai_status {
    SLAI_OK = 0,
    SLAI_ERR_INVALID_ARG = 1,
    SLAI_ERR_UNSUPPORTED_FORMAT = 2,
    SLAI_ERR_SHAPE = 3,
    SLAI_ERR_CUDA = 4,
    SLAI_ERR_NCCL = 5,
    SLAI_ERR_TIMEOUT = 6,
    SLAI_ERR_OOM = 7
};

/* GGML tensor type ids as stored in GGUF files (gguf.rs:20-60).  F32, Q8_0, Q4_K, Q5_K and Q6_K have kernels of
 * their own.  The legacy formats (quantization.rs:47-199) are accepted at upload: Q4_0 and Q5_0 are re-expressed
 * exactly as Q8_0 blocks (same f16 scale, quant - 8 / - 16 as int8), Q4_1, Q5_1 and Q8_K are dequantised to dense f32
 * with the reference's rounding (what the reference does with tensors its quantised kernels do not take,
 * gguf.rs:148-162).  F16 has no path: SLAI_ERR_UNSUPPORTED_FORMAT. */
enum slai_format {
    SLAI_FMT_F32 = 0,
    SLAI_FMT_F16 = 1,
    SLAI_FMT_Q4_0 = 2,
    SLAI_FMT_Q4_1 = 3,
    SLAI_FMT_Q5_0 = 6,
    SLAI_FMT_Q5_1 = 7,
    SLAI_FMT_Q8_0 = 8,
    SLAI_FMT_Q4_K = 12,
    SLAI_FMT_Q5_K = 13,
    SLAI_FMT_Q6_K = 14,
    SLAI_FMT_Q8_K = 15
};

enum slai_kv_dtype { SLAI_KV_F32 = 0, SLAI_KV_F16 = 1 };

/* ---- context: LlmOps::new / LlmContext::begin_submission / submit (context.rs:47-96) ---------------- */
int slai_ctx_create(int device, slai_ctx** out);
int slai_ctx_destroy(slai_ctx* ctx);
/* backend.synchronize() (chat_llama2.rs:222-223); blocking.  Also reports SLAI_ERR_TIMEOUT when a bounded wait
 * inside a kernel (weight ring, grid barrier) ran out since the last call: every device-side wait has an
 * iteration limit and raises a flag instead of hanging. */
int slai_ctx_sync(slai_ctx* ctx);
/* Rounds a device-side wait polls before it gives up (default 2^20, about a second).  No counterpart in the
 * reference, whose dispatches never wait on one another.  Applies to launches described after the call; a host
 * that supervises its ranks itself can shorten it to detect a missing peer sooner.  rounds >= 16. */
int slai_ctx_set_wait_limit(slai_ctx* ctx, uint32_t rounds);
const char* slai_last_error_string(slai_ctx* ctx);
void* slai_ctx_stream(slai_ctx* ctx); /* the cudaStream_t all work of this context is enqueued on */
int slai_device_count(void);
/* Device name and number of SMs of the context's GPU. */
int slai_ctx_device_info(slai_ctx* ctx, char* name, int name_len, int* sm_count);
/* Free and total bytes of the context's GPU (cudaMemGetInfo). */
int slai_ctx_mem_info(slai_ctx* ctx, size_t* free_bytes, size_t* total_bytes);

/* ---- buffers: Backend::write_buffer / read_buffer (slang-hal, used at chat_llama2.rs:180-230) ------- */
int slai_malloc(slai_ctx* ctx, size_t bytes, void** d_out);
int slai_free(slai_ctx* ctx, void* d_ptr);
int slai_memset(slai_ctx* ctx, void* d_ptr, int value, size_t bytes);
int slai_write_buffer(slai_ctx* ctx, void* d_dst, const void* h_src, size_t bytes); /* async if pinned  */
int slai_read_buffer(slai_ctx* ctx, void* h_dst, const void* d_src, size_t bytes);  /* blocking         */
int slai_malloc_host(slai_ctx* ctx, size_t bytes, void** h_out); /* pinned host memory */
int slai_free_host(slai_ctx* ctx, void* h_ptr);

/* ---- recorded passes: B::Encoder / begin_pass ... submit (context.rs:63-96, slai-bench main.rs:199-219) -- */
/* The reference records operator launches into an encoder and submits them together.  Here: every operator call
 * between `slai_pass_begin` and `slai_pass_end` is recorded (CUDA stream capture) instead of run; the recorded pass
 * is replayed with `slai_pass_launch` (`times` back-to-back replays, no host work between the kernels).
 * Calls that allocate or block (matrix creation, reads, the first `slai_attention` at a new size) cannot be
 * recorded: run the sequence once eagerly first.  Arguments are frozen at record time; buffers a recorded call
 * uses must stay allocated until the pass is destroyed, and nothing may be freed or copied synchronously while
 * recording (both synchronise the device, which ends the recording with an error). */
typedef struct slai_pass slai_pass;
int slai_pass_begin(slai_ctx* ctx);
int slai_pass_end(slai_ctx* ctx, slai_pass** out);
int slai_pass_launch(slai_ctx* ctx, slai_pass* pass, int times);
int slai_pass_destroy(slai_ctx* ctx, slai_pass* pass);

/* ---- tensor-parallel group (no counterpart in the reference, which runs a model on one device) ---------- */
/* One process (or thread) per GPU, one context each.  Rank 0 asks for an id, the host program hands the 128 bytes
 * to the other ranks by any means (a torch.distributed / MPI broadcast, a file), every rank calls slai_tp_init
 * (collective: returns when all ranks have joined).  Models created afterwards with tp_size > 1 in their
 * configuration take weights that the caller has already sharded (column-parallel matrices by rows, row-parallel
 * ones by columns on block boundaries, each rank its own KV heads) and exchange one sum
 * of `dim` floats after the attention output projection and after the FFN down projection of every layer
 * (NCCL all-reduce over NVLink on the context's stream). */
#define SLAI_TP_ID_BYTES 128
int slai_tp_unique_id(slai_ctx* ctx, void* h_id);                             /* h_id: SLAI_TP_ID_BYTES bytes out */
int slai_tp_init(slai_ctx* ctx, const void* h_id, int rank, int size);        /* blocking, collective */
int slai_tp_all_reduce_sum(slai_ctx* ctx, const float* d_in, float* d_out, int64_t n); /* in place allowed */
int slai_tp_shutdown(slai_ctx* ctx);                                          /* blocking, collective */
/* Optional: exchange over peer memory instead of NCCL (ranks = separate processes on GPUs of one NVLink domain).
 * Every rank exports its exchange region (a CUDA IPC handle), the host program gathers the handles of all ranks in
 * rank order and every rank attaches them; the host must let all ranks finish attaching (a barrier) before the
 * first decode call.  Models created afterwards store their partial rows straight into the peers' regions from the
 * producing kernel's epilogue and sum them in the consuming kernel's prologue (no collective kernel).  Waits on
 * peers are bounded: a rank that never arrives shows up as SLAI_ERR_TIMEOUT at the next slai_ctx_sync. */
#define SLAI_TP_HANDLE_BYTES 64
int slai_tp_peer_export(slai_ctx* ctx, void* h_handle);            /* h_handle: SLAI_TP_HANDLE_BYTES bytes out; blocking */
int slai_tp_peer_attach(slai_ctx* ctx, const void* h_handles);     /* tp_size x SLAI_TP_HANDLE_BYTES bytes, rank order */
/* The two operators a caller that assembles its own sharded transformer needs (the models use them internally; no
 * counterpart in the reference).  `index` numbers the exchanges inside one token (0 .. per_token-1, alternating
 * buffers), slai_tp_token_tick starts a new token.
 *  - slai_gemv_quant_partial: this rank's partial of a row-parallel product, W v (+ d_resid on rank 0), stored as
 *    (value, tag) pairs into every rank's region from the kernel's epilogue.
 *  - slai_gemv_quant_reduced: d_out = W rmsnorm(s) where s = the sum over ranks of exchange `index`, formed while
 *    the kernel stages its input (bounded polls on the tags); s is also left in d_sum_out (ncols floats). */
int slai_tp_token_tick(slai_ctx* ctx);
int slai_gemv_quant_partial(slai_ctx* ctx, const slai_qmatrix* w, const float* d_v, const float* d_resid, int index, int per_token);
int slai_gemv_quant_reduced(slai_ctx* ctx, float* d_out, const slai_qmatrix* w, const float* d_norm_w, float eps, int index,
                            int per_token, float* d_sum_out);
/* Single-GPU stand-in for slai_tp_peer_attach: the context's own region plays every rank's, and the caller plays
 * the ranks one after another by calling again with another `rank` (2 <= ranks <= 8).  For checking the exchange
 * arithmetic and its time-out path without a second GPU; models do not use it. */
int slai_tp_peer_loopback(slai_ctx* ctx, int ranks, int rank);

/* ---- stream timing: the GPU timestamp queries of crates/slai-bench/src/main.rs:198,221-242 ---------- */
int slai_timer_start(slai_ctx* ctx);          /* records an event on the stream */
int slai_timer_stop(slai_ctx* ctx, float* ms); /* records, waits, returns elapsed milliseconds; blocking */

/* ---- quantized matrices: GgufTensor::to_gpu_matrix (gguf.rs:133-194,357-366) ------------------------- */
/* `h_blocks`: nrows rows of (ncols / block_elems) GGUF blocks, row-major, exactly the file's bytes.
 * On upload the blocks are re-laid-out tile-major (16 rows x one K step per contiguous block, same byte
 * count up to zero padding of the last tile) so that the kernels stream them with bulk copies; F32 is
 * kept dense.  Unlike the reference there is no "dequantise when the block count is odd" fallback:
 * every shape with ncols % block_elems == 0 stays quantized. */
int slai_qmatrix_create(slai_ctx* ctx, int fmt, int64_t nrows, int64_t ncols, const void* h_blocks, size_t nbytes,
                        slai_qmatrix** out);
/* Same, with the raw blocks already in device memory. */
int slai_qmatrix_create_from_device(slai_ctx* ctx, int fmt, int64_t nrows, int64_t ncols, const void* d_blocks,
                                    size_t nbytes, slai_qmatrix** out);
int slai_qmatrix_destroy(slai_qmatrix* m);
int slai_qmatrix_shape(const slai_qmatrix* m, int* fmt, int64_t* nrows, int64_t* ncols); /* quantized_matrix.rs:25-38 */
size_t slai_qmatrix_device_bytes(const slai_qmatrix* m);
/* Bit-exact dump of the dequantised values, row-major f32 [nrows*ncols]: Block*::dequantize()
 * (quantization.rs:38-41,214-243,275-316,347-378) evaluated on the GPU with the reference's rounding. */
int slai_qmatrix_dequantize(slai_ctx* ctx, const slai_qmatrix* m, float* d_out);
/* One dequantised row (the embedding lookup `token_embd.column(token)`, chat_llama2.rs:186-188). */
int slai_qmatrix_dequantize_row(slai_ctx* ctx, const slai_qmatrix* m, int64_t row, float* d_out);

/* Synthetic weights generated on the device: raw GGUF blocks of `fmt` quantised from N(0, std) floats
 * drawn from a counter-based generator keyed by `seed`.  `d_blocks` must hold
 * nrows * ncols / block_elems * block_bytes bytes.  No counterpart in the reference (it has no quantiser);
 * used by the benchmarks to build model-sized inputs without host-side generation. */
int slai_synth_blocks(slai_ctx* ctx, int fmt, int64_t nrows, int64_t ncols, uint64_t seed, float std, void* d_blocks);
/* N(0, std) f32 values from the same generator. */
int slai_synth_normal_f32(slai_ctx* ctx, float* d_out, int64_t n, uint64_t seed, float std);

/* ---- GemvQuant::launch (ops/gemv_quant.rs:206-312); LlmContext::matmul_quant_assign (context.rs:355-369)
 * d_out[b*M + i] = sum_k W[i][k] * d_v[b*K + k] for b < n_batch (1 <= n_batch <= 8).  A batch of 2..8 vectors is served
 * by one pass over a quantised matrix (d_v 16-byte aligned); dense f32 matrices take the vectors one by one.  The batched
 * kernel keeps per-chunk partial sums in the context's scratch buffer, grown on demand: inside a recorded pass
 * (slai_pass_begin) call it only after one eager call of the same matrix shape and batch. */
int slai_gemv_quant(slai_ctx* ctx, float* d_out, const slai_qmatrix* w, const float* d_v, int n_batch);
/* The feed-forward front half of a Llama layer as one kernel: out[hidden] = silu(Wgate n(x)) * (Wup n(x)) with
 * n = RmsNorm by `d_norm_w` and `eps` (null weights: x is used as it is).  Replaces the four dispatches RmsNorm::launch,
 * two GemvQuant::launch and Silu::launch of crates/slai/src/models/llama2/transformer.rs:356-361; both matrices must
 * share one quantised format and shape. */
int slai_ffn_gate_up(slai_ctx* ctx, float* d_out, const slai_qmatrix* w_gate, const slai_qmatrix* w_up, const float* d_x,
                     const float* d_norm_w, float eps);

/* ---- RmsNorm::launch (ops/rms_norm.rs:35-67): out[i] = (x[i] * rsqrt(mean(x^2) + eps)) * w[i] -------- */
int slai_rms_norm(slai_ctx* ctx, float* d_out, const float* d_x, const float* d_w, int64_t n, float eps);

/* ---- RoPE::launch (ops/rope.rs:45-85); RoPEConfig {head_size, kv_dim, pos, base_freq} (:28-33).
 * variant 0 = Original (adjacent pairs), 1 = Neox.  q has q_len floats, k has at least kv_dim. */
int slai_rope(slai_ctx* ctx, int variant, float* d_q, int64_t q_len, float* d_k, int head_size, int kv_dim, int pos,
              float base_freq);

/* ---- Silu::launch (ops/silu.rs:24-48): h1[i] = h2[i] * h1[i] / (1 + exp(-h1[i])) --------------------- */
int slai_silu_gate(slai_ctx* ctx, float* d_h1_inout, const float* d_h2, int64_t n);

/* ---- Unary::launch / launch_inplace (ops/unary.rs:171-306); `op` indexes UnaryOp (:11-35) in order:
 * 0 Abs 1 Sgn 2 Neg 3 Step 4 Elu 5 Gelu 6 GeluQuick 7 Silu 8 Tanh 9 Sin 10 Cos 11 Relu 12 Sigmoid
 * 13 HardSigmoid 14 Sqr 15 Sqrt 16 Log 17 LeakyRelu 18 Clamp 19 Scale 20 AddScalar.  dst may equal src. */
int slai_unary(slai_ctx* ctx, int op, float* d_dst, const float* d_src, int64_t n, const float args4[4]);

/* ---- SoftMax::launch_cols (ops/softmax.rs:22-40): softmax of each of `ncols` columns of `nrows`
 * floats, column c starting at d_m + c*col_stride. */
int slai_softmax_cols(slai_ctx* ctx, float* d_m, int64_t nrows, int64_t ncols, int64_t col_stride);

/* ---- LayerNorm::launch_cols (ops/layernorm.rs:25-60) followed by the caller's gamma/beta
 * (models/gpt2/cpu.rs:235-240): y = (x-mean)/sqrt(var+eps) [* gamma + beta]; gamma/beta may be NULL. */
int slai_layernorm(slai_ctx* ctx, float* d_out, const float* d_x, int64_t n, float eps, const float* d_gamma,
                   const float* d_beta);

/* ---- LlmContext::add_assign / mul_assign / copy (context.rs:428-469,660-673) ------------------------- */
int slai_add_assign(slai_ctx* ctx, float* d_a, const float* d_b, int64_t n);
int slai_mul_assign(slai_ctx* ctx, float* d_a, const float* d_b, int64_t n);
int slai_copy(slai_ctx* ctx, float* d_dst, const float* d_src, int64_t n);

/* ---- Sampler::sample_argmax (models/sampler.rs:55-57): first maximal index, on the device ------------ */
/* Sampler::sample (models/sampler.rs:33-131) with the uniform random number `coin` in [0, 1) given by the caller;
 * d_logits is overwritten with the probabilities, as in the reference. */
int slai_sample(slai_ctx* ctx, float* d_logits, int64_t n, float temperature, float topp, float coin, int32_t* d_token_out);
int slai_argmax(slai_ctx* ctx, const float* d_v, int64_t n, int32_t* d_index_out);

/* ---- BatchedMultiqueryAttention::launch (ops/batched_multiquery_attention.rs:32-100) ------------------
 * Same field order as BatchedMultiqueryAttentionParams (:17-29). */
typedef struct slai_attn_params {
    uint32_t seq_len, kv_dim, kv_mul, n_heads, head_size, pos;
    uint32_t _padding[2];
} slai_attn_params;
/* Caches are position-major as in the reference: position t occupies kv_dim consecutive elements
 * (f32 or f16), head h at offset h*head_size.  The score buffer of the reference (`attn`) is internal. */
int slai_attention(slai_ctx* ctx, const slai_attn_params* p, const float* d_q, const void* d_key_cache,
                   const void* d_value_cache, int kv_dtype, float* d_xb);
/* ---- slai_attention for callers that may not allocate.  This entry point has no counterpart in the
 * reference (whose scratch tensors always come from its backend's allocator).
 * Same arguments and result as slai_attention, but the call itself requests no memory (no cudaMalloc / cudaFree,
 * no allocating library routine): the split partials, the per-head tickets and the position scalar live in a
 * device array that is part of the library image, SLAI_ATTENTION_STATIC_MAX_SCRATCH_BYTES + 4352 bytes per GPU
 * that loads the library, held until the process exits.  It is meant for hosts that receive their device memory
 * once and must stay off the driver allocator afterwards (an engine that partitions the GPU among its subsystems,
 * a serving loop whose latency path may not synchronise on cudaMalloc / cudaFree).
 *  - Shapes whose partials at the LAST position of the cache (seq_len - 1) exceed the array are rejected with
 *    SLAI_ERR_SHAPE and a message naming both sizes, from the first call on; use slai_attention for those.
 *  - The first call on a device does the one-time set-up: it resolves the array's device address
 *    (cudaGetSymbolAddress, with that device current) and is the first launch of the attention kernel there, so the
 *    CUDA runtime loads the kernel image and applies its shared-memory attribute then (the runtime may take
 *    device memory of its own for that).  Make that first call before starting any stream capture; from the second
 *    call on the free device memory does not change.  The caller's current device is left as it was.
 *  - All calls share the one array and it keeps the last call's contents: each call re-zeroes the tickets it uses
 *    and rewrites the position; two calls whose kernels overlap on the GPU (different contexts / streams on the
 *    same device) race on it.  Calls on one context are ordered by its stream and are safe. */
#define SLAI_ATTENTION_STATIC_MAX_SCRATCH_BYTES (4u << 20)
int slai_attention_static(slai_ctx* ctx, const slai_attn_params* p, const float* d_q, const void* d_key_cache,
                          const void* d_value_cache, int kv_dtype, float* d_xb);
/* Writes the kv_dim-float vectors k and v into position `pos` of the caches (the reference lets the K/V
 * GEMVs write into `key_cache.column(pos)` directly, transformer.rs:329-334). */
int slai_kv_append(slai_ctx* ctx, void* d_key_cache, void* d_value_cache, int kv_dtype, const float* d_k,
                   const float* d_v, int kv_dim, int pos);

/* ---- Llama-2 family: Llama2Config (models/llama2/cpu.rs:46-67), Llama2::launch (transformer.rs:316-381) */
typedef struct slai_llama_config {
    int32_t dim, hidden_dim, n_layers, n_q_heads, n_kv_heads, vocab_size, seq_len;
    float rope_base_freq, rms_norm_eps;
    int32_t rope_variant; /* 0 Original, 1 Neox (models/llama2/mod.rs:27-32) */
    int32_t kv_dtype;     /* slai_kv_dtype; the reference keeps f32 (transformer.rs:87-106) */
    int32_t tp_rank, tp_size; /* 0,1 unless sharded with slai_tp */
} slai_llama_config;

enum slai_llama_weight { /* tensor names at transformer.rs:208-219,270-283 */
    SLAI_W_TOKEN_EMBD = 0, SLAI_W_OUT_NORM = 1, SLAI_W_OUTPUT = 2, SLAI_W_ATTN_NORM = 3, SLAI_W_Q = 4,
    SLAI_W_K = 5, SLAI_W_V = 6, SLAI_W_O = 7, SLAI_W_FFN_NORM = 8, SLAI_W_GATE = 9, SLAI_W_UP = 10,
    SLAI_W_DOWN = 11, SLAI_W_BQ = 12, SLAI_W_BK = 13, SLAI_W_BV = 14
};

int slai_llama_create(slai_ctx* ctx, const slai_llama_config* cfg, slai_llama** out); /* Llama2State::new */
int slai_llama_destroy(slai_llama* m);
/* Llama2Weights::from_gguf (transformer.rs:201-297): matrices are attached (not copied; they must outlive
 * the model), f32 vectors (norm weights, biases, the f32 embedding table) are copied from the host. */
int slai_llama_set_matrix(slai_llama* m, int weight_id, int layer, const slai_qmatrix* w);
int slai_llama_set_f32(slai_llama* m, int weight_id, int layer, const float* h_data, int64_t n);
/* Same with the data already on the device (copied device-to-device). */
int slai_llama_set_f32_device(slai_llama* m, int weight_id, int layer, const float* d_data, int64_t n);
/* One token through Llama2::launch.  ChatLlama2::forward_logits (chat_llama2.rs:163-240): embedding
 * lookup, all layers, logits.  `h_logits` (vocab floats) may be NULL; `next_token` (greedy argmax computed
 * on the device) may be NULL.  Blocking when either output is requested. */
int slai_llama_decode(slai_llama* m, int32_t token, int32_t pos, float* h_logits, int32_t* next_token);
/* `n` greedy steps without host round trips: feeds each argmax back as the next token, starting with
 * `token` at `pos`; writes the n produced token ids to h_tokens.  Blocking. */
int slai_llama_generate(slai_llama* m, int32_t token, int32_t pos, int32_t n, int32_t* h_tokens);
/* The same loop with Sampler::sample (models/sampler.rs:33-54) on the device instead of greedy: temperature 0 is
 * greedy; topp outside (0, 1) draws from the whole distribution.  The uniform number of step i is the top 24 bits of
 * splitmix64(seed + i) / 2^24 (the reference draws from an unseeded generator, :43). */
int slai_llama_generate_sampled(slai_llama* m, int32_t token, int32_t pos, int32_t n, float temperature, float topp, uint64_t seed,
                                int32_t* h_tokens);
/* Prompt processing: tokens[0..n) at positions pos0.. ; fills the KV cache.  If h_last_logits is non-NULL
 * it receives the logits of the last prompt token.  Blocking.  The reference feeds the prompt through its decode step
 * token by token (chat_llama2.rs:109-115); here prompts of 16 tokens or more go through every matrix together as
 * GEMMs on the tensor cores (quantised matrices whose column count is a multiple of 64; a sharded model sums the
 * partial products of its row-parallel matrices with the group's all-reduce, so every rank must make the call),
 * shorter ones and everything else through the decode step as there.  Same results within 1e-3 relative L2. */
int slai_llama_prefill(slai_llama* m, const int32_t* h_tokens, int32_t n, int32_t pos0, float* h_last_logits);
/* Several sequences decoded together (no counterpart in the reference, whose Llama2State holds one sequence:
 * models/llama2/transformer.rs:16-44): `slai_llama_batch_reserve` gives the model `n_seq` (1..8; 0 frees them) further KV
 * caches and activation rows; `slai_llama_decode_batch` takes one token of each of the first `n_seq` sequences, token
 * h_tokens[b] at position h_pos[b] of sequence b's own cache, and reads every weight matrix once for all of them (the
 * operator sequence of Llama2::launch, transformer.rs:316-381, on n_seq columns).  A negative position leaves that
 * sequence out of the step.  h_logits (n_seq x vocab floats) and h_next (the greedy choice per sequence) may be NULL.
 * Blocking.  Models without q/k/v biases, not sharded.  Per sequence the results equal slai_llama_decode's within 1e-3
 * relative L2. */
int slai_llama_batch_reserve(slai_llama* m, int32_t n_seq);
int slai_llama_decode_batch(slai_llama* m, int32_t n_seq, const int32_t* h_tokens, const int32_t* h_pos, float* h_logits, int32_t* h_next);
/* Debug/test access to Llama2State vectors: 0 x, 1 xb, 2 q, 3 hb, 4 logits.  Blocking. */
int slai_llama_read_state(slai_llama* m, int which, float* h_out, int64_t n);
/* Test access to the KV cache of one layer: positions 0..n_pos as f32, position-major like the reference's cache
 * (h_keys / h_values: n_pos x kv_dim floats).  Blocking. */
int slai_llama_read_kv(slai_llama* m, int layer, int n_pos, float* h_keys, float* h_values);
/* Where a decode step spends its device time.  Classes (index of `us` / `launches`): 0 everything else (embedding,
 * rotation, sampling, collectives, gaps between kernels), 1 norm + q/k/v GEMV + RoPE + cache append, 2 attention,
 * 3 output projection + residual, 4 norm + gate/up GEMV + SiLU, 5 down projection + residual, 6 final norm + logits
 * GEMV.  The step runs once outside the replayed graph, kernel after kernel (no overlap between launches), with events
 * around each launch: the sum is therefore larger than the time of a replayed step; the split is what it is for.  It
 * is a real step: position `pos` of the KV cache is written.  Replaces reading the reference's per-dispatch GPU
 * timestamps (crates/slai/src/models/llama2/transformer.rs:316-381 runs each operator as its own dispatch). */
typedef struct slai_llama_stats_t {
    float us_total;
    float us[7];
    int32_t launches[7];
} slai_llama_stats_t;
int slai_llama_stats(slai_llama* m, int32_t token, int32_t pos, slai_llama_stats_t* out);
/* Number of kernel launches issued for the last decoded token. */
int slai_llama_launches_per_token(const slai_llama* m);

/* ---- GPT-2: Gpt2Params (models/gpt2/cpu.rs:19-35), Transformer::forward (:225-383) -------------------- */
typedef struct slai_gpt2_config {
    int32_t n_vocab, n_seq, n_embd, n_head, n_layer, ff_len;
    float layernorm_eps;
    int32_t kv_dtype;
} slai_gpt2_config;

enum slai_gpt2_weight { /* fields of Gpt2Layer / Gpt2Model (models/gpt2/cpu.rs:66-112) */
    SLAI_G_WTE = 0, SLAI_G_WPE = 1, SLAI_G_LNF_G = 2, SLAI_G_LNF_B = 3, SLAI_G_LN1_G = 4, SLAI_G_LN1_B = 5,
    SLAI_G_W_QKV = 6, SLAI_G_B_QKV = 7, SLAI_G_W_PROJ = 8, SLAI_G_B_PROJ = 9, SLAI_G_LN2_G = 10,
    SLAI_G_LN2_B = 11, SLAI_G_W_FC = 12, SLAI_G_B_FC = 13, SLAI_G_W_FCPROJ = 14, SLAI_G_B_FCPROJ = 15
};

int slai_gpt2_create(slai_ctx* ctx, const slai_gpt2_config* cfg, slai_gpt2** out);
int slai_gpt2_destroy(slai_gpt2* m);
int slai_gpt2_set_matrix(slai_gpt2* m, int weight_id, int layer, const slai_qmatrix* w);
int slai_gpt2_set_f32(slai_gpt2* m, int weight_id, int layer, const float* h_data, int64_t n);
int slai_gpt2_decode(slai_gpt2* m, int32_t token, int32_t pos, float* h_logits, int32_t* next_token);
int slai_gpt2_generate(slai_gpt2* m, int32_t token, int32_t pos, int32_t n, int32_t* h_tokens);
/* As slai_llama_prefill: prompts of 16 tokens or more go through every matrix together as tensor-core GEMMs (quantised
 * matrices whose column count is a multiple of 64, head size a multiple of 8), the rest token by token. */
int slai_gpt2_prefill(slai_gpt2* m, const int32_t* h_tokens, int32_t n, int32_t pos0, float* h_last_logits);

#ifdef __cplusplus
}
#endif
#endif /* SLAI_B200_H */
