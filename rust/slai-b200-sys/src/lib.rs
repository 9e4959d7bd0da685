//! Raw FFI bindings to `libslai_b200.so` (C ABI: `include/slai_b200.h`).
//! One declaration per exported function; the safe wrappers over them live in the `slai-b200` crate next to this one.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_void};

macro_rules! opaque { ($($n:ident),*) => { $(#[repr(C)] pub struct $n { _private: [u8; 0] })* } }
opaque!(slai_ctx, slai_qmatrix, slai_llama, slai_gpt2, slai_pass);

pub const SLAI_OK: i32 = 0;
pub const SLAI_ERR_INVALID_ARG: i32 = 1;
pub const SLAI_ERR_UNSUPPORTED_FORMAT: i32 = 2;
pub const SLAI_ERR_SHAPE: i32 = 3;
pub const SLAI_ERR_CUDA: i32 = 4;
pub const SLAI_ERR_NCCL: i32 = 5;
pub const SLAI_ERR_TIMEOUT: i32 = 6;
pub const SLAI_ERR_OOM: i32 = 7;

/// Same field order as `BatchedMultiqueryAttentionParams` (crates/slai/src/ops/batched_multiquery_attention.rs:17-29).
#[repr(C)]
#[derive(Copy, Clone, Debug, Default)]
pub struct slai_attn_params { pub seq_len: u32, pub kv_dim: u32, pub kv_mul: u32, pub n_heads: u32, pub head_size: u32, pub pos: u32, pub _padding: [u32; 2] }

/// `Llama2Config` (crates/slai/src/models/llama2/cpu.rs:46-67) plus the cache type.
#[repr(C)]
#[derive(Copy, Clone, Debug)]
pub struct slai_llama_config { pub dim: i32, pub hidden_dim: i32, pub n_layers: i32, pub n_q_heads: i32, pub n_kv_heads: i32, pub vocab_size: i32,
    pub seq_len: i32, pub rope_base_freq: f32, pub rms_norm_eps: f32, pub rope_variant: i32, pub kv_dtype: i32, pub tp_rank: i32, pub tp_size: i32 }

/// Device time of one decode step per kernel class (see `slai_llama_stats` in the C header).
#[repr(C)]
#[derive(Copy, Clone, Debug, Default)]
pub struct slai_llama_stats_t { pub us_total: f32, pub us: [f32; 7], pub launches: [i32; 7] }

/// `Gpt2Params` (crates/slai/src/models/gpt2/cpu.rs:19-35).
#[repr(C)]
#[derive(Copy, Clone, Debug)]
pub struct slai_gpt2_config { pub n_vocab: i32, pub n_seq: i32, pub n_embd: i32, pub n_head: i32, pub n_layer: i32, pub ff_len: i32, pub layernorm_eps: f32, pub kv_dtype: i32 }

extern "C" {
    pub fn slai_ctx_create(device: i32, out: *mut *mut slai_ctx) -> i32;
    pub fn slai_ctx_destroy(ctx: *mut slai_ctx) -> i32;
    pub fn slai_ctx_sync(ctx: *mut slai_ctx) -> i32;
    pub fn slai_ctx_set_wait_limit(ctx: *mut slai_ctx, rounds: u32) -> i32;
    pub fn slai_tp_token_tick(ctx: *mut slai_ctx) -> i32;
    pub fn slai_gemv_quant_partial(ctx: *mut slai_ctx, w: *const slai_qmatrix, d_v: *const f32, d_resid: *const f32, index: i32, per_token: i32) -> i32;
    pub fn slai_gemv_quant_reduced(ctx: *mut slai_ctx, d_out: *mut f32, w: *const slai_qmatrix, d_norm_w: *const f32, eps: f32, index: i32, per_token: i32, d_sum_out: *mut f32) -> i32;
    pub fn slai_tp_peer_loopback(ctx: *mut slai_ctx, ranks: i32, rank: i32) -> i32;
    pub fn slai_last_error_string(ctx: *mut slai_ctx) -> *const c_char;
    pub fn slai_ctx_stream(ctx: *mut slai_ctx) -> *mut c_void;
    pub fn slai_device_count() -> i32;
    pub fn slai_ctx_mem_info(ctx: *mut slai_ctx, free_bytes: *mut usize, total_bytes: *mut usize) -> i32;
    pub fn slai_ctx_device_info(ctx: *mut slai_ctx, name: *mut c_char, name_len: i32, sm_count: *mut i32) -> i32;
    pub fn slai_malloc(ctx: *mut slai_ctx, bytes: usize, d_out: *mut *mut c_void) -> i32;
    pub fn slai_free(ctx: *mut slai_ctx, d_ptr: *mut c_void) -> i32;
    pub fn slai_memset(ctx: *mut slai_ctx, d_ptr: *mut c_void, value: i32, bytes: usize) -> i32;
    pub fn slai_write_buffer(ctx: *mut slai_ctx, d_dst: *mut c_void, h_src: *const c_void, bytes: usize) -> i32;
    pub fn slai_read_buffer(ctx: *mut slai_ctx, h_dst: *mut c_void, d_src: *const c_void, bytes: usize) -> i32;
    pub fn slai_malloc_host(ctx: *mut slai_ctx, bytes: usize, h_out: *mut *mut c_void) -> i32;
    pub fn slai_free_host(ctx: *mut slai_ctx, h_ptr: *mut c_void) -> i32;
    pub fn slai_pass_begin(ctx: *mut slai_ctx) -> i32;
    pub fn slai_pass_end(ctx: *mut slai_ctx, out: *mut *mut slai_pass) -> i32;
    pub fn slai_pass_launch(ctx: *mut slai_ctx, pass: *mut slai_pass, times: i32) -> i32;
    pub fn slai_pass_destroy(ctx: *mut slai_ctx, pass: *mut slai_pass) -> i32;
    pub fn slai_tp_unique_id(ctx: *mut slai_ctx, h_id: *mut c_void) -> i32;
    pub fn slai_tp_init(ctx: *mut slai_ctx, h_id: *const c_void, rank: i32, size: i32) -> i32;
    pub fn slai_tp_all_reduce_sum(ctx: *mut slai_ctx, d_in: *const f32, d_out: *mut f32, n: i64) -> i32;
    pub fn slai_tp_shutdown(ctx: *mut slai_ctx) -> i32;
    pub fn slai_tp_peer_export(ctx: *mut slai_ctx, h_handle: *mut c_void) -> i32;
    pub fn slai_tp_peer_attach(ctx: *mut slai_ctx, h_handles: *const c_void) -> i32;
    pub fn slai_timer_start(ctx: *mut slai_ctx) -> i32;
    pub fn slai_timer_stop(ctx: *mut slai_ctx, ms: *mut f32) -> i32;
    pub fn slai_qmatrix_create(ctx: *mut slai_ctx, fmt: i32, nrows: i64, ncols: i64, h_blocks: *const c_void, nbytes: usize, out: *mut *mut slai_qmatrix) -> i32;
    pub fn slai_qmatrix_create_from_device(ctx: *mut slai_ctx, fmt: i32, nrows: i64, ncols: i64, d_blocks: *const c_void, nbytes: usize, out: *mut *mut slai_qmatrix) -> i32;
    pub fn slai_qmatrix_destroy(m: *mut slai_qmatrix) -> i32;
    pub fn slai_qmatrix_shape(m: *const slai_qmatrix, fmt: *mut i32, nrows: *mut i64, ncols: *mut i64) -> i32;
    pub fn slai_qmatrix_device_bytes(m: *const slai_qmatrix) -> usize;
    pub fn slai_qmatrix_dequantize(ctx: *mut slai_ctx, m: *const slai_qmatrix, d_out: *mut f32) -> i32;
    pub fn slai_qmatrix_dequantize_row(ctx: *mut slai_ctx, m: *const slai_qmatrix, row: i64, d_out: *mut f32) -> i32;
    pub fn slai_synth_blocks(ctx: *mut slai_ctx, fmt: i32, nrows: i64, ncols: i64, seed: u64, std: f32, d_blocks: *mut c_void) -> i32;
    pub fn slai_synth_normal_f32(ctx: *mut slai_ctx, d_out: *mut f32, n: i64, seed: u64, std: f32) -> i32;
    pub fn slai_gemv_quant(ctx: *mut slai_ctx, d_out: *mut f32, w: *const slai_qmatrix, d_v: *const f32, n_batch: i32) -> i32;
    pub fn slai_ffn_gate_up(ctx: *mut slai_ctx, d_out: *mut f32, w_gate: *const slai_qmatrix, w_up: *const slai_qmatrix, d_x: *const f32, d_norm_w: *const f32, eps: f32) -> i32;
    pub fn slai_rms_norm(ctx: *mut slai_ctx, d_out: *mut f32, d_x: *const f32, d_w: *const f32, n: i64, eps: f32) -> i32;
    pub fn slai_rope(ctx: *mut slai_ctx, variant: i32, d_q: *mut f32, q_len: i64, d_k: *mut f32, head_size: i32, kv_dim: i32, pos: i32, base_freq: f32) -> i32;
    pub fn slai_silu_gate(ctx: *mut slai_ctx, d_h1_inout: *mut f32, d_h2: *const f32, n: i64) -> i32;
    pub fn slai_unary(ctx: *mut slai_ctx, op: i32, d_dst: *mut f32, d_src: *const f32, n: i64, args4: *const f32) -> i32;
    pub fn slai_softmax_cols(ctx: *mut slai_ctx, d_m: *mut f32, nrows: i64, ncols: i64, col_stride: i64) -> i32;
    pub fn slai_layernorm(ctx: *mut slai_ctx, d_out: *mut f32, d_x: *const f32, n: i64, eps: f32, d_gamma: *const f32, d_beta: *const f32) -> i32;
    pub fn slai_add_assign(ctx: *mut slai_ctx, d_a: *mut f32, d_b: *const f32, n: i64) -> i32;
    pub fn slai_mul_assign(ctx: *mut slai_ctx, d_a: *mut f32, d_b: *const f32, n: i64) -> i32;
    pub fn slai_copy(ctx: *mut slai_ctx, d_dst: *mut f32, d_src: *const f32, n: i64) -> i32;
    pub fn slai_argmax(ctx: *mut slai_ctx, d_v: *const f32, n: i64, d_index_out: *mut i32) -> i32;
    pub fn slai_attention(ctx: *mut slai_ctx, p: *const slai_attn_params, d_q: *const f32, d_key_cache: *const c_void, d_value_cache: *const c_void, kv_dtype: i32, d_xb: *mut f32) -> i32;
    pub fn slai_attention_static(ctx: *mut slai_ctx, p: *const slai_attn_params, d_q: *const f32, d_key_cache: *const c_void, d_value_cache: *const c_void, kv_dtype: i32, d_xb: *mut f32) -> i32;
    pub fn slai_kv_append(ctx: *mut slai_ctx, d_key_cache: *mut c_void, d_value_cache: *mut c_void, kv_dtype: i32, d_k: *const f32, d_v: *const f32, kv_dim: i32, pos: i32) -> i32;
    pub fn slai_llama_create(ctx: *mut slai_ctx, cfg: *const slai_llama_config, out: *mut *mut slai_llama) -> i32;
    pub fn slai_llama_destroy(m: *mut slai_llama) -> i32;
    pub fn slai_llama_set_matrix(m: *mut slai_llama, weight_id: i32, layer: i32, w: *const slai_qmatrix) -> i32;
    pub fn slai_llama_set_f32(m: *mut slai_llama, weight_id: i32, layer: i32, h_data: *const f32, n: i64) -> i32;
    pub fn slai_llama_set_f32_device(m: *mut slai_llama, weight_id: i32, layer: i32, d_data: *const f32, n: i64) -> i32;
    pub fn slai_llama_decode(m: *mut slai_llama, token: i32, pos: i32, h_logits: *mut f32, next_token: *mut i32) -> i32;
    pub fn slai_llama_generate(m: *mut slai_llama, token: i32, pos: i32, n: i32, h_tokens: *mut i32) -> i32;
    pub fn slai_llama_generate_sampled(m: *mut slai_llama, token: i32, pos: i32, n: i32, temperature: f32, topp: f32, seed: u64, h_tokens: *mut i32) -> i32;
    pub fn slai_sample(ctx: *mut slai_ctx, d_logits: *mut f32, n: i64, temperature: f32, topp: f32, coin: f32, d_token_out: *mut i32) -> i32;
    pub fn slai_llama_prefill(m: *mut slai_llama, h_tokens: *const i32, n: i32, pos0: i32, h_last_logits: *mut f32) -> i32;
    pub fn slai_llama_read_state(m: *mut slai_llama, which: i32, h_out: *mut f32, n: i64) -> i32;
    pub fn slai_llama_read_kv(m: *mut slai_llama, layer: i32, n_pos: i32, h_keys: *mut f32, h_values: *mut f32) -> i32;
    pub fn slai_llama_stats(m: *mut slai_llama, token: i32, pos: i32, out: *mut slai_llama_stats_t) -> i32;
    pub fn slai_llama_batch_reserve(m: *mut slai_llama, n_seq: i32) -> i32;
    pub fn slai_llama_decode_batch(m: *mut slai_llama, n_seq: i32, h_tokens: *const i32, h_pos: *const i32, h_logits: *mut f32,
                                   h_next: *mut i32) -> i32;
    pub fn slai_llama_launches_per_token(m: *const slai_llama) -> i32;
    pub fn slai_gpt2_create(ctx: *mut slai_ctx, cfg: *const slai_gpt2_config, out: *mut *mut slai_gpt2) -> i32;
    pub fn slai_gpt2_destroy(m: *mut slai_gpt2) -> i32;
    pub fn slai_gpt2_set_matrix(m: *mut slai_gpt2, weight_id: i32, layer: i32, w: *const slai_qmatrix) -> i32;
    pub fn slai_gpt2_set_f32(m: *mut slai_gpt2, weight_id: i32, layer: i32, h_data: *const f32, n: i64) -> i32;
    pub fn slai_gpt2_decode(m: *mut slai_gpt2, token: i32, pos: i32, h_logits: *mut f32, next_token: *mut i32) -> i32;
    pub fn slai_gpt2_generate(m: *mut slai_gpt2, token: i32, pos: i32, n: i32, h_tokens: *mut i32) -> i32;
    pub fn slai_gpt2_prefill(m: *mut slai_gpt2, h_tokens: *const i32, n: i32, pos0: i32, h_last_logits: *mut f32) -> i32;
}

/// Error type the safe wrappers return in place of `B::Error`.
#[derive(Debug)]
pub enum B200Error { InvalidArg(String), UnsupportedFormat(String), Shape(String), Cuda(String), Nccl(String), Timeout(String), Oom(String) }

/// Maps a status code to `Result`, attaching the library's message.
pub unsafe fn check(code: i32, ctx: *mut slai_ctx) -> Result<(), B200Error> {
    if code == SLAI_OK { return Ok(()); }
    let msg = std::ffi::CStr::from_ptr(slai_last_error_string(ctx)).to_string_lossy().into_owned();
    Err(match code {
        SLAI_ERR_INVALID_ARG => B200Error::InvalidArg(msg),
        SLAI_ERR_UNSUPPORTED_FORMAT => B200Error::UnsupportedFormat(msg),
        SLAI_ERR_SHAPE => B200Error::Shape(msg),
        SLAI_ERR_NCCL => B200Error::Nccl(msg),
        SLAI_ERR_TIMEOUT => B200Error::Timeout(msg),
        SLAI_ERR_OOM => B200Error::Oom(msg),
        _ => B200Error::Cuda(msg),
    })
}
