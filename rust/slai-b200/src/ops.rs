//! The operators of `crates/slai/src/ops/*.rs` on a `B200`.  Each `launch` keeps the reference's argument order with
//! the `shapes` argument dropped; the structs are unit types (the reference's hold compiled shader pipelines).
use crate::{sys, B200Error, B200Pass, GpuQuantMatrix, KvDtype, View, ViewMut, B200};
use std::os::raw::c_void;

/// `GemvQuant<B>` (ops/gemv_quant.rs:101-131).
#[derive(Default)]
pub struct GemvQuant;
impl GemvQuant {
    pub fn new(_backend: &B200) -> Self {
        GemvQuant
    }
    /// `GemvQuant::launch` (ops/gemv_quant.rs:206-312): queues `out = m * v`.
    pub fn launch<'b>(&self, backend: &B200, _pass: &mut B200Pass, out: impl Into<ViewMut<'b, f32>>, m: &GpuQuantMatrix, v: impl Into<View<'b, f32>>) -> Result<(), B200Error> {
        let (out, v) = (out.into(), v.into());
        let [rows, cols] = m.shape();
        if cols == 0 || v.len() % cols != 0 || out.len() != rows * (v.len() / cols) {
            return Err(B200Error::Shape(format!("gemv: {rows}x{cols} matrix, vector of {}, output of {}", v.len(), out.len())));
        }
        backend.check(unsafe { sys::slai_gemv_quant(backend.h, out.ptr, m.h, v.ptr, (v.len() / cols) as i32) })
    }
}

/// `RmsNormConfig` (ops/rms_norm.rs:15-21).
#[repr(C)]
#[derive(Copy, Clone, Debug)]
pub struct RmsNormConfig {
    pub nudge_factor: f32,
    pub _padding: [f32; 3],
}
/// `RmsNorm<B>` (ops/rms_norm.rs:11-13).
#[derive(Default)]
pub struct RmsNorm;
impl RmsNorm {
    /// `RmsNorm::launch` (ops/rms_norm.rs:35-66): `result = value / sqrt(mean(value^2) + nudge) * weight`.
    pub fn launch<'b>(&self, backend: &B200, _pass: &mut B200Pass, config: &RmsNormConfig, result: impl Into<ViewMut<'b, f32>>, value: impl Into<View<'b, f32>>,
                      weight: impl Into<View<'b, f32>>) -> Result<(), B200Error> {
        let (result, value, weight) = (result.into(), value.into(), weight.into());
        if result.len() != value.len() || weight.len() != value.len() {
            return Err(B200Error::Shape("rms_norm: lengths differ".into()));
        }
        backend.check(unsafe { sys::slai_rms_norm(backend.h, result.ptr, value.ptr, weight.ptr, value.len() as i64, config.nudge_factor) })
    }
}

/// `RoPEVariant` (ops/rope.rs:9-16).
#[repr(i32)]
#[derive(Copy, Clone, Debug, PartialEq, Eq)]
pub enum RoPEVariant {
    Original = 0,
    Neox = 1,
}
/// `RoPEConfig` (ops/rope.rs:28-33).
#[repr(C)]
#[derive(Copy, Clone, Debug)]
pub struct RoPEConfig {
    pub head_size: u32,
    pub kv_dim: u32,
    pub pos: u32,
    pub base_freq: f32,
}
/// `RoPE<B>` (ops/rope.rs:19-25).
#[derive(Default)]
pub struct RoPE;
impl RoPE {
    /// `RoPE::launch` (ops/rope.rs:45-86).  Where the reference asserts (odd lengths, `len(q) < len(k)`) this returns
    /// `B200Error::Shape`.
    pub fn launch<'b>(&self, backend: &B200, _pass: &mut B200Pass, variant: RoPEVariant, config: &RoPEConfig, in_out_q: impl Into<ViewMut<'b, f32>>,
                      in_out_k: impl Into<ViewMut<'b, f32>>) -> Result<(), B200Error> {
        let (q, k) = (in_out_q.into(), in_out_k.into());
        if k.len() < config.kv_dim as usize {
            return Err(B200Error::Shape("rope: k shorter than kv_dim".into()));
        }
        backend.check(unsafe { sys::slai_rope(backend.h, variant as i32, q.ptr, q.len() as i64, k.ptr, config.head_size as i32, config.kv_dim as i32, config.pos as i32, config.base_freq) })
    }
}

/// `Silu<B>` (ops/silu.rs:11-13).
#[derive(Default)]
pub struct Silu;
impl Silu {
    /// `Silu::launch` (ops/silu.rs:24-48): `h1 = h2 * h1 / (1 + exp(-h1))`.
    pub fn launch<'b>(&self, backend: &B200, _pass: &mut B200Pass, in_out_h1: impl Into<ViewMut<'b, f32>>, in_h2: impl Into<View<'b, f32>>) -> Result<(), B200Error> {
        let (h1, h2) = (in_out_h1.into(), in_h2.into());
        if h1.len() != h2.len() {
            return Err(B200Error::Shape("silu: lengths differ".into()));
        }
        backend.check(unsafe { sys::slai_silu_gate(backend.h, h1.ptr, h2.ptr, h1.len() as i64) })
    }
}

/// `UnaryOp` (ops/unary.rs:11-35), same order.
#[repr(i32)]
#[derive(Copy, Clone, Debug, PartialEq, Eq)]
pub enum UnaryOp {
    Abs = 0, Sgn, Neg, Step, Elu, Gelu, GeluQuick, Silu, Tanh, Sin, Cos, Relu, Sigmoid, HardSigmoid, Sqr, Sqrt, Log, LeakyRelu, Clamp, Scale, AddScalar,
}
/// `Unary<B>` (ops/unary.rs:112-118).
#[derive(Default)]
pub struct Unary;
impl Unary {
    /// `Unary::launch_inplace` (ops/unary.rs:171-223).
    pub fn launch_inplace<'b>(&self, backend: &B200, _pass: &mut B200Pass, op: UnaryOp, in_out: impl Into<ViewMut<'b, f32>>, args: [f32; 4]) -> Result<(), B200Error> {
        let x = in_out.into();
        backend.check(unsafe { sys::slai_unary(backend.h, op as i32, x.ptr, x.ptr, x.len() as i64, args.as_ptr()) })
    }
    /// `Unary::launch` (ops/unary.rs:225-282).
    pub fn launch<'b>(&self, backend: &B200, _pass: &mut B200Pass, op: UnaryOp, dest: impl Into<ViewMut<'b, f32>>, src: impl Into<View<'b, f32>>, args: [f32; 4]) -> Result<(), B200Error> {
        let (d, s) = (dest.into(), src.into());
        if d.len() != s.len() {
            return Err(B200Error::Shape("unary: lengths differ".into()));
        }
        backend.check(unsafe { sys::slai_unary(backend.h, op as i32, d.ptr, s.ptr, s.len() as i64, args.as_ptr()) })
    }
}

/// `SoftMax<B>` (ops/softmax.rs:11-13).
#[derive(Default)]
pub struct SoftMax;
impl SoftMax {
    /// `SoftMax::launch_cols` (ops/softmax.rs:22-40): soft-max of each of `ncols` columns of `nrows` elements, columns
    /// `col_stride` elements apart.
    pub fn launch_cols<'b>(&self, backend: &B200, _pass: &mut B200Pass, in_out_mat: impl Into<ViewMut<'b, f32>>, nrows: usize, ncols: usize, col_stride: usize) -> Result<(), B200Error> {
        let m = in_out_mat.into();
        if ncols > 0 && (ncols - 1) * col_stride + nrows > m.len() {
            return Err(B200Error::Shape("softmax: matrix larger than the buffer".into()));
        }
        backend.check(unsafe { sys::slai_softmax_cols(backend.h, m.ptr, nrows as i64, ncols as i64, col_stride as i64) })
    }
}

/// `LayerNorm<B>` (ops/layernorm.rs:11-14).
#[derive(Default)]
pub struct LayerNorm;
impl LayerNorm {
    /// `LayerNorm::launch_cols` on one column (ops/layernorm.rs:25-60); `eps` is the reference CPU twin's 1e-5
    /// (ops/layernorm.rs:105) unless the caller says otherwise.  `gamma` / `beta` fold in the scale and shift the
    /// reference's caller applies next (models/gpt2/cpu.rs:239-240).
    pub fn launch_cols<'b>(&self, backend: &B200, _pass: &mut B200Pass, output: impl Into<ViewMut<'b, f32>>, input: impl Into<View<'b, f32>>, eps: f32,
                           gamma: Option<View<'b, f32>>, beta: Option<View<'b, f32>>) -> Result<(), B200Error> {
        let (o, i) = (output.into(), input.into());
        if o.len() != i.len() {
            return Err(B200Error::Shape("layernorm: lengths differ".into()));
        }
        let g = gamma.map_or(std::ptr::null(), |v| v.ptr);
        let b = beta.map_or(std::ptr::null(), |v| v.ptr);
        backend.check(unsafe { sys::slai_layernorm(backend.h, o.ptr, i.ptr, i.len() as i64, eps, g, b) })
    }
}

/// `BatchedMultiqueryAttentionParams` (ops/batched_multiquery_attention.rs:17-29).
pub type BatchedMultiqueryAttentionParams = sys::slai_attn_params;

/// `BatchedMultiqueryAttention<B>` (ops/batched_multiquery_attention.rs:13-15).
#[derive(Default)]
pub struct BatchedMultiqueryAttention;
impl BatchedMultiqueryAttention {
    /// `BatchedMultiqueryAttention::launch` (ops/batched_multiquery_attention.rs:32-100).  The reference's `attn`
    /// scratch tensor and `params_gpu` copy are internal here; the caches are position-major `[seq_len][kv_dim]`
    /// (transformer.rs:87-106) in `kv_dtype` elements.
    pub fn launch<'b>(&self, backend: &B200, _pass: &mut B200Pass, params: &BatchedMultiqueryAttentionParams, q: impl Into<View<'b, f32>>, key_cache: *const c_void,
                      value_cache: *const c_void, kv_dtype: KvDtype, xb: impl Into<ViewMut<'b, f32>>) -> Result<(), B200Error> {
        let (q, xb) = (q.into(), xb.into());
        let dim = (params.n_heads * params.head_size) as usize;
        if q.len() < dim || xb.len() < dim {
            return Err(B200Error::Shape("attention: q / xb shorter than n_heads * head_size".into()));
        }
        backend.check(unsafe { sys::slai_attention(backend.h, params, q.ptr, key_cache, value_cache, kv_dtype as i32, xb.ptr) })
    }
}

/// The convenience methods of `LlmContext` (context.rs:205-501,760-797) that the decode path uses.
pub struct LlmContext<'a> {
    pub backend: &'a B200,
    pub gemv_quant: GemvQuant,
    pub rms_norm: RmsNorm,
    pub rope: RoPE,
    pub silu: Silu,
    pub unary: Unary,
    pub softmax: SoftMax,
    pub layernorm: LayerNorm,
    pub attention: BatchedMultiqueryAttention,
}
impl<'a> LlmContext<'a> {
    pub fn new(backend: &'a B200) -> Self {
        LlmContext { backend, gemv_quant: GemvQuant, rms_norm: RmsNorm, rope: RoPE, silu: Silu, unary: Unary, softmax: SoftMax, layernorm: LayerNorm, attention: BatchedMultiqueryAttention }
    }
    /// `LlmContext::matmul_quant_assign` (context.rs:355-369).
    pub fn matmul_quant_assign<'b>(&self, out: impl Into<ViewMut<'b, f32>>, a: &GpuQuantMatrix, b: impl Into<View<'b, f32>>) -> Result<(), B200Error> {
        let mut pass = self.backend.begin_submission();
        self.gemv_quant.launch(self.backend, &mut pass, out, a, b)
    }
    /// The feed-forward front half of a Llama layer as one kernel: `out = silu(w_gate n(x)) * (w_up n(x))`, `n` = RmsNorm by
    /// `norm_w` (None: `x` as it is).  Stands for the four dispatches of transformer.rs:356-361.
    pub fn ffn_gate_up<'b>(&self, out: impl Into<ViewMut<'b, f32>>, w_gate: &GpuQuantMatrix, w_up: &GpuQuantMatrix, x: impl Into<View<'b, f32>>,
                           norm_w: Option<View<'b, f32>>, eps: f32) -> Result<(), B200Error> {
        let (out, x) = (out.into(), x.into());
        let [rows, cols] = w_gate.shape();
        if w_up.shape() != [rows, cols] || x.len() != cols || out.len() != rows || norm_w.map_or(false, |w| w.len() != cols) {
            return Err(B200Error::Shape("ffn_gate_up: shapes differ".into()));
        }
        let nw = norm_w.map_or(std::ptr::null(), |w| w.ptr);
        self.backend.check(unsafe { sys::slai_ffn_gate_up(self.backend.h, out.ptr, w_gate.h, w_up.h, x.ptr, nw, eps) })
    }
    /// `LlmContext::add_assign` (context.rs:428-441).
    pub fn add_assign<'b>(&self, a: impl Into<ViewMut<'b, f32>>, b: impl Into<View<'b, f32>>) -> Result<(), B200Error> {
        let (a, b) = (a.into(), b.into());
        if a.len() != b.len() {
            return Err(B200Error::Shape("add_assign: lengths differ".into()));
        }
        self.backend.check(unsafe { sys::slai_add_assign(self.backend.h, a.ptr, b.ptr, a.len() as i64) })
    }
    /// `LlmContext::mul_assign` (context.rs:456-469).
    pub fn mul_assign<'b>(&self, a: impl Into<ViewMut<'b, f32>>, b: impl Into<View<'b, f32>>) -> Result<(), B200Error> {
        let (a, b) = (a.into(), b.into());
        if a.len() != b.len() {
            return Err(B200Error::Shape("mul_assign: lengths differ".into()));
        }
        self.backend.check(unsafe { sys::slai_mul_assign(self.backend.h, a.ptr, b.ptr, a.len() as i64) })
    }
    /// `LlmContext::copy` (context.rs:660-673).
    pub fn copy<'b>(&self, dst: impl Into<ViewMut<'b, f32>>, src: impl Into<View<'b, f32>>) -> Result<(), B200Error> {
        let (d, s) = (dst.into(), src.into());
        if d.len() != s.len() {
            return Err(B200Error::Shape("copy: lengths differ".into()));
        }
        self.backend.check(unsafe { sys::slai_copy(self.backend.h, d.ptr, s.ptr, s.len() as i64) })
    }
    /// Appends this position's key and value rows to the caches (the reference writes the K / V GEMV outputs straight
    /// into column `pos`, transformer.rs:329-334).
    pub fn kv_append<'b>(&self, key_cache: *mut c_void, value_cache: *mut c_void, kv_dtype: KvDtype, k: impl Into<View<'b, f32>>, v: impl Into<View<'b, f32>>, pos: u32) -> Result<(), B200Error> {
        let (k, v) = (k.into(), v.into());
        if k.len() != v.len() {
            return Err(B200Error::Shape("kv_append: k and v differ in length".into()));
        }
        self.backend.check(unsafe { sys::slai_kv_append(self.backend.h, key_cache, value_cache, kv_dtype as i32, k.ptr, v.ptr, k.len() as i32, pos as i32) })
    }
}
