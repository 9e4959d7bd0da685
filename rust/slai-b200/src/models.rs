//! Model handles: the decode step of `Llama2::launch` (crates/slai/src/models/llama2/transformer.rs:316-381) and of the
//! GPT-2 twin (models/gpt2/cpu.rs:225-383) as one call each, with state and weights owned by the library.
use crate::{sys, B200Error, GpuQuantMatrix, B200};
use std::ptr;

pub use sys::slai_gpt2_config as Gpt2Config;
pub use sys::slai_llama_config as Llama2Config;
pub use sys::slai_llama_stats_t as Llama2Stats;

/// Tensor names of `Llama2Weights::from_gguf` (transformer.rs:208-219,270-283).
#[repr(i32)]
#[derive(Copy, Clone, Debug, PartialEq, Eq)]
pub enum LlamaWeight {
    TokenEmbd = 0, OutNorm = 1, Output = 2, AttnNorm = 3, Q = 4, K = 5, V = 6, O = 7, FfnNorm = 8, Gate = 9, Up = 10, Down = 11, BiasQ = 12, BiasK = 13, BiasV = 14,
}

/// `Llama2State` + `Llama2Weights` + `Llama2::launch` behind one handle.
pub struct Llama2<'a> {
    backend: &'a B200,
    h: *mut sys::slai_llama,
    vocab: usize,
}
impl<'a> Llama2<'a> {
    pub fn new(backend: &'a B200, config: &Llama2Config) -> Result<Self, B200Error> {
        let mut h = ptr::null_mut();
        backend.check(unsafe { sys::slai_llama_create(backend.h, config, &mut h) })?;
        Ok(Llama2 { backend, h, vocab: config.vocab_size as usize })
    }
    /// The matrix stays owned by the caller and must outlive the model.
    pub fn set_matrix(&mut self, which: LlamaWeight, layer: i32, m: &'a GpuQuantMatrix<'a>) -> Result<(), B200Error> {
        self.backend.check(unsafe { sys::slai_llama_set_matrix(self.h, which as i32, layer, m.h) })
    }
    pub fn set_f32(&mut self, which: LlamaWeight, layer: i32, data: &[f32]) -> Result<(), B200Error> {
        self.backend.check(unsafe { sys::slai_llama_set_f32(self.h, which as i32, layer, data.as_ptr(), data.len() as i64) })
    }
    /// `ChatLlama2::forward_logits(pos, token, &mut logits)` (slai-chat/src/chat_llama2.rs:163-240); returns the greedy
    /// token (`Sampler::sample_argmax`, models/sampler.rs:34-36) computed on the device.
    pub fn forward_logits(&mut self, pos: u32, token: u32, logits: &mut [f32]) -> Result<u32, B200Error> {
        if logits.len() != self.vocab {
            return Err(B200Error::Shape("forward_logits: logits must hold vocab_size floats".into()));
        }
        let mut next = 0i32;
        self.backend.check(unsafe { sys::slai_llama_decode(self.h, token as i32, pos as i32, logits.as_mut_ptr(), &mut next) })?;
        Ok(next as u32)
    }
    /// Feeds `tokens` at positions `pos0..`; prompts of 16 tokens or more run as tensor-core GEMMs.
    pub fn prefill(&mut self, tokens: &[i32], pos0: u32, last_logits: Option<&mut [f32]>) -> Result<(), B200Error> {
        let p = last_logits.map_or(ptr::null_mut(), |l| l.as_mut_ptr());
        self.backend.check(unsafe { sys::slai_llama_prefill(self.h, tokens.as_ptr(), tokens.len() as i32, pos0 as i32, p) })
    }
    /// `n` greedy tokens starting from `token` at `pos`, token selection on the device.
    pub fn generate(&mut self, token: u32, pos: u32, n: usize) -> Result<Vec<i32>, B200Error> {
        let mut out = vec![0i32; n];
        self.backend.check(unsafe { sys::slai_llama_generate(self.h, token as i32, pos as i32, n as i32, out.as_mut_ptr()) })?;
        Ok(out)
    }
    /// The same loop with `Sampler::sample` (models/sampler.rs:33-54: temperature, nucleus) on the device.
    pub fn generate_sampled(&mut self, token: u32, pos: u32, n: usize, temperature: f32, topp: f32, seed: u64) -> Result<Vec<i32>, B200Error> {
        let mut out = vec![0i32; n];
        self.backend.check(unsafe { sys::slai_llama_generate_sampled(self.h, token as i32, pos as i32, n as i32, temperature, topp, seed, out.as_mut_ptr()) })?;
        Ok(out)
    }
    /// KV caches and activation rows for `n_seq` (1..8) sequences decoded together; 0 frees them.
    pub fn batch_reserve(&mut self, n_seq: usize) -> Result<(), B200Error> {
        self.backend.check(unsafe { sys::slai_llama_batch_reserve(self.h, n_seq as i32) })
    }
    /// One token of each sequence: `tokens[b]` at `positions[b]` of sequence b's own cache (a negative position leaves the
    /// sequence out of the step); every weight matrix is read once for all of them.  `logits`, when given, holds
    /// `tokens.len() * vocab_size` floats.  Returns the greedy token per sequence.
    pub fn decode_batch(&mut self, tokens: &[i32], positions: &[i32], logits: Option<&mut [f32]>) -> Result<Vec<i32>, B200Error> {
        if tokens.len() != positions.len() || logits.as_ref().map_or(false, |l| l.len() != tokens.len() * self.vocab) {
            return Err(B200Error::Shape("decode_batch: one position per token, vocab_size logits per sequence".into()));
        }
        let mut next = vec![0i32; tokens.len()];
        let p = logits.map_or(ptr::null_mut(), |l| l.as_mut_ptr());
        self.backend.check(unsafe {
            sys::slai_llama_decode_batch(self.h, tokens.len() as i32, tokens.as_ptr(), positions.as_ptr(), p, next.as_mut_ptr())
        })?;
        Ok(next)
    }
    /// Device time of one decode step per kernel class.
    pub fn stats(&mut self, token: u32, pos: u32) -> Result<Llama2Stats, B200Error> {
        let mut st = Llama2Stats::default();
        self.backend.check(unsafe { sys::slai_llama_stats(self.h, token as i32, pos as i32, &mut st) })?;
        Ok(st)
    }
}
impl<'a> Drop for Llama2<'a> {
    fn drop(&mut self) {
        unsafe { sys::slai_llama_destroy(self.h) };
    }
}

/// Fields of `Gpt2Layer` / `Gpt2Model` (models/gpt2/cpu.rs:66-112).
#[repr(i32)]
#[derive(Copy, Clone, Debug, PartialEq, Eq)]
pub enum Gpt2Weight {
    Wte = 0, Wpe = 1, LnfG = 2, LnfB = 3, Ln1G = 4, Ln1B = 5, WQkv = 6, BQkv = 7, WProj = 8, BProj = 9, Ln2G = 10, Ln2B = 11, WFc = 12, BFc = 13, WFcProj = 14, BFcProj = 15,
}

pub struct Gpt2<'a> {
    backend: &'a B200,
    h: *mut sys::slai_gpt2,
    vocab: usize,
}
impl<'a> Gpt2<'a> {
    pub fn new(backend: &'a B200, config: &Gpt2Config) -> Result<Self, B200Error> {
        let mut h = ptr::null_mut();
        backend.check(unsafe { sys::slai_gpt2_create(backend.h, config, &mut h) })?;
        Ok(Gpt2 { backend, h, vocab: config.n_vocab as usize })
    }
    pub fn set_matrix(&mut self, which: Gpt2Weight, layer: i32, m: &'a GpuQuantMatrix<'a>) -> Result<(), B200Error> {
        self.backend.check(unsafe { sys::slai_gpt2_set_matrix(self.h, which as i32, layer, m.h) })
    }
    pub fn set_f32(&mut self, which: Gpt2Weight, layer: i32, data: &[f32]) -> Result<(), B200Error> {
        self.backend.check(unsafe { sys::slai_gpt2_set_f32(self.h, which as i32, layer, data.as_ptr(), data.len() as i64) })
    }
    /// `Transformer::forward(token, pos)` (models/gpt2/cpu.rs:225-383) plus the greedy token.
    pub fn forward(&mut self, token: u32, pos: u32, logits: &mut [f32]) -> Result<u32, B200Error> {
        if logits.len() != self.vocab {
            return Err(B200Error::Shape("forward: logits must hold n_vocab floats".into()));
        }
        let mut next = 0i32;
        self.backend.check(unsafe { sys::slai_gpt2_decode(self.h, token as i32, pos as i32, logits.as_mut_ptr(), &mut next) })?;
        Ok(next as u32)
    }
    pub fn generate(&mut self, token: u32, pos: u32, n: usize) -> Result<Vec<i32>, B200Error> {
        let mut out = vec![0i32; n];
        self.backend.check(unsafe { sys::slai_gpt2_generate(self.h, token as i32, pos as i32, n as i32, out.as_mut_ptr()) })?;
        Ok(out)
    }
}
impl<'a> Drop for Gpt2<'a> {
    fn drop(&mut self) {
        unsafe { sys::slai_gpt2_destroy(self.h) };
    }
}
