"""Llama-2-family and GPT-2 decoders on the C ABI, mirroring slai's model types.

`Llama2Config` / `Llama2` follow crates/slai/src/models/llama2/cpu.rs:46-143 and transformer.rs:16-381;
`Gpt2Params` / `Gpt2` follow crates/slai/src/models/gpt2/cpu.rs:19-383.  Weight tensors carry the GGUF names
the reference loads (transformer.rs:208-219,270-283).  The synthetic builders stand in for checkpoints
(none is available offline): seeded normal weights quantised to GGUF blocks.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib, synth
from ._lib import Gpt2Config as _CGpt2Config, LlamaConfig as _CLlamaConfig, KV_F16, KV_F32
from .ops import Backend, GpuQuantMatrix, GpuVector

LLAMA_W = dict(token_embd=0, out_norm=1, output=2, attn_norm=3, wq=4, wk=5, wv=6, wo=7, ffn_norm=8, w_gate=9, w_up=10,
               w_down=11, bq=12, bk=13, bv=14)
GPT2_W = dict(wte=0, wpe=1, lnf_g=2, lnf_b=3, ln1_g=4, ln1_b=5, w_qkv=6, b_qkv=7, w_proj=8, b_proj=9, ln2_g=10, ln2_b=11,
              w_fc=12, b_fc=13, w_fcproj=14, b_fcproj=15)
LLAMA_MATRICES = ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")
GPT2_MATRICES = ("w_qkv", "w_proj", "w_fc", "w_fcproj")


@dataclass
class Llama2Config:
    dim: int
    hidden_dim: int
    n_layers: int
    n_q_heads: int
    n_kv_heads: int
    vocab_size: int
    seq_len: int
    rope_base_freq: float = 10000.0
    rms_norm_eps: float = 1e-5
    rope_variant: int = 0
    kv_dtype: int = KV_F16

    @property
    def head_size(self):
        return self.dim // self.n_q_heads

    @property
    def kv_dim(self):
        return self.dim * self.n_kv_heads // self.n_q_heads

    def matrix_shapes(self):
        return dict(wq=(self.dim, self.dim), wk=(self.kv_dim, self.dim), wv=(self.kv_dim, self.dim), wo=(self.dim, self.dim),
                    w_gate=(self.hidden_dim, self.dim), w_up=(self.hidden_dim, self.dim), w_down=(self.dim, self.hidden_dim))

    def weight_bytes_per_token(self, fmt: int, out_fmt: int) -> int:
        """Packed weight bytes streamed per decoded token (all layers + the logits matrix)."""
        per = sum(r * c for r, c in self.matrix_shapes().values())
        bpw, bpo = synth.BITS_PER_WEIGHT[fmt], synth.BITS_PER_WEIGHT[out_fmt]
        return int(self.n_layers * per * bpw / 8 + self.vocab_size * self.dim * bpo / 8)

    def kv_bytes_at(self, pos: int) -> int:
        esz = 2 if self.kv_dtype == KV_F16 else 4
        return 2 * self.n_layers * self.kv_dim * esz * (pos + 1)


TINY_LLAMA = Llama2Config(dim=288, hidden_dim=768, n_layers=6, n_q_heads=6, n_kv_heads=6, vocab_size=32000, seq_len=256)
LLAMA2_7B = Llama2Config(dim=4096, hidden_dim=11008, n_layers=32, n_q_heads=32, n_kv_heads=32, vocab_size=32000, seq_len=4096)
LLAMA2_70B = Llama2Config(dim=8192, hidden_dim=28672, n_layers=80, n_q_heads=64, n_kv_heads=8, vocab_size=32000, seq_len=4096)


class Llama2:
    """Llama2State + Llama2Weights + Llama2::launch behind one handle."""

    def __init__(self, backend: Backend, config: Llama2Config, tp_rank: int = 0, tp_size: int = 1):
        """`config` is the whole model's; with tp_size > 1 (after `slai_b200.tp.join_group`) the matrices attached
        must be this rank's shards (`slai_b200.tp.shard_shapes`)."""
        self.backend, self.config = backend, config
        self.tp_rank, self.tp_size = tp_rank, tp_size
        c = _CLlamaConfig(config.dim, config.hidden_dim, config.n_layers, config.n_q_heads, config.n_kv_heads, config.vocab_size,
                          config.seq_len, config.rope_base_freq, config.rms_norm_eps, config.rope_variant, config.kv_dtype,
                          tp_rank, tp_size)
        h = C.c_void_p()
        backend.check(backend.lib.slai_llama_create(backend.h, C.byref(c), C.byref(h)))
        self.h = h
        self._keep = []

    def set_matrix(self, name: str, layer: int, m: GpuQuantMatrix):
        self._keep.append(m)
        self.backend.check(self.backend.lib.slai_llama_set_matrix(self.h, LLAMA_W[name], layer, m.h))

    def set_f32(self, name: str, layer: int, data):
        if isinstance(data, GpuVector):
            self.backend.check(self.backend.lib.slai_llama_set_f32_device(self.h, LLAMA_W[name], layer, C.c_void_p(data.ptr), data.n))
            return
        a = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        self.backend.check(self.backend.lib.slai_llama_set_f32(self.h, LLAMA_W[name], layer, a.ctypes.data_as(C.c_void_p), a.size))

    def forward_logits(self, pos: int, token: int, logits: np.ndarray | None = None):
        """`ChatLlama2::forward_logits(pos, token, &mut logits)` (chat_llama2.rs:163-240)."""
        if logits is None:
            logits = np.empty(self.config.vocab_size, dtype=np.float32)
        nxt = C.c_int32()
        self.backend.check(self.backend.lib.slai_llama_decode(self.h, token, pos, logits.ctypes.data_as(C.c_void_p), C.byref(nxt)))
        return logits, nxt.value

    def decode_async(self, token: int, pos: int):
        """One token, nothing read back (enqueue only)."""
        self.backend.check(self.backend.lib.slai_llama_decode(self.h, token, pos, None, None))

    def decode_into(self, token: int, pos: int, logits_ptr: int):
        """One token; logits copied into host memory at `logits_ptr` (e.g. pinned); returns the greedy token."""
        nxt = C.c_int32()
        self.backend.check(self.backend.lib.slai_llama_decode(self.h, token, pos, C.c_void_p(logits_ptr), C.byref(nxt)))
        return nxt.value

    def generate(self, token: int, pos: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int32)
        self.backend.check(self.backend.lib.slai_llama_generate(self.h, token, pos, n, out.ctypes.data_as(C.c_void_p)))
        return out

    def generate_sampled(self, token: int, pos: int, n: int, temperature: float, topp: float, seed: int) -> np.ndarray:
        """The generate loop with `Sampler::sample` (models/sampler.rs:33-54) on the device; see `sample_coin`."""
        out = np.empty(n, dtype=np.int32)
        self.backend.check(self.backend.lib.slai_llama_generate_sampled(self.h, token, pos, n, temperature, topp, seed,
                                                                        out.ctypes.data_as(C.c_void_p)))
        return out

    def prefill(self, tokens, pos0: int = 0, want_logits: bool = False):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.config.vocab_size, dtype=np.float32) if want_logits else None
        self.backend.check(self.backend.lib.slai_llama_prefill(self.h, t.ctypes.data_as(C.c_void_p), t.size, pos0,
                                                               logits.ctypes.data_as(C.c_void_p) if want_logits else None))
        return logits

    def batch_reserve(self, n_seq: int):
        """KV caches and activation rows for `n_seq` (1..8) sequences decoded together; 0 frees them."""
        self.backend.check(self.backend.lib.slai_llama_batch_reserve(self.h, n_seq))

    def decode_batch(self, tokens, positions, want_logits: bool = True):
        """One token of each sequence (tokens[b] at positions[b] of sequence b's own cache; a negative position leaves the
        sequence out): every weight matrix is read once for all of them.  Returns (logits [n, vocab] or None, greedy ids [n])."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        if t.shape != p.shape or t.ndim != 1:
            raise ValueError("decode_batch: tokens and positions must be vectors of the same length")
        logits = np.empty((t.size, self.config.vocab_size), dtype=np.float32) if want_logits else None
        nxt = np.empty(t.size, dtype=np.int32)
        self.backend.check(self.backend.lib.slai_llama_decode_batch(self.h, t.size, t.ctypes.data_as(C.c_void_p), p.ctypes.data_as(C.c_void_p),
                                                                    logits.ctypes.data_as(C.c_void_p) if want_logits else None,
                                                                    nxt.ctypes.data_as(C.c_void_p)))
        return logits, nxt

    def stats(self, token: int, pos: int) -> dict:
        """Device microseconds per kernel class of one (real) decode step run kernel after kernel outside the graph."""
        from ._lib import LlamaStats
        st = LlamaStats()
        self.backend.check(self.backend.lib.slai_llama_stats(self.h, token, pos, C.byref(st)))
        out = {"total_us": float(st.us_total)}
        for i, name in enumerate(LlamaStats.CLASSES):
            out[name] = {"us": float(st.us[i]), "launches": int(st.launches[i])}
        return out

    def read_kv(self, layer: int, n_pos: int):
        """Keys and values of one layer for positions 0..n_pos, each [n_pos, kv_dim] f32 (test access)."""
        kvd = self.config.kv_dim // max(self.tp_size, 1) if hasattr(self, "tp_size") else self.config.kv_dim
        k = np.empty((n_pos, kvd), dtype=np.float32)
        v = np.empty((n_pos, kvd), dtype=np.float32)
        self.backend.check(self.backend.lib.slai_llama_read_kv(self.h, layer, n_pos, k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p)))
        return k, v

    def read_state(self, which: str) -> np.ndarray:
        idx = dict(x=0, xb=1, q=2, hb=3, logits=4)[which]
        n = dict(x=self.config.dim, xb=self.config.dim, q=self.config.dim, hb=self.config.hidden_dim, logits=self.config.vocab_size)[which]
        out = np.empty(n, dtype=np.float32)
        self.backend.check(self.backend.lib.slai_llama_read_state(self.h, idx, out.ctypes.data_as(C.c_void_p), n))
        return out

    def launches_per_token(self) -> int:
        return int(self.backend.lib.slai_llama_launches_per_token(self.h))

    def close(self):
        if getattr(self, "h", None) and self.backend.h:
            self.backend.lib.slai_llama_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sample_coin(seed: int, step: int) -> float:
    """The uniform number the device sampler uses at step `step`: top 24 bits of splitmix64(seed + step) / 2^24."""
    m = (1 << 64) - 1
    x = (seed + step + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    x ^= x >> 31
    return float((x >> 40) & 0xFFFFFF) / 16777216.0


def _seed(base: int, name: str, layer: int) -> list[int]:
    return [base, sum(ord(ch) * (i + 1) for i, ch in enumerate(name)), layer + 1]


def synthetic_llama_host(config: Llama2Config, fmt: int, out_fmt: int | None = None, seed: int = 0, std: float = 0.02,
                         embd_std: float = 0.02):
    """Seeded weights on the host: {(name, layer): GGUF block bytes or f32 array}.  Norm weights are 1."""
    out_fmt = fmt if out_fmt is None else out_fmt
    w = {}
    for l in range(config.n_layers):
        for name, (r, c) in config.matrix_shapes().items():
            w[(name, l)] = synth.quantize(fmt, synth.normal_matrix(_seed(seed, name, l), r, c, std))
        w[("attn_norm", l)] = np.ones(config.dim, dtype=np.float32)
        w[("ffn_norm", l)] = np.ones(config.dim, dtype=np.float32)
    w[("token_embd", -1)] = synth.normal_matrix(_seed(seed, "token_embd", -1), config.vocab_size, config.dim, embd_std)
    w[("out_norm", -1)] = np.ones(config.dim, dtype=np.float32)
    w[("output", -1)] = synth.quantize(out_fmt, synth.normal_matrix(_seed(seed, "output", -1), config.vocab_size, config.dim, std))
    return w


def llama_from_host(backend: Backend, config: Llama2Config, weights: dict, fmt: int, out_fmt: int | None = None) -> Llama2:
    out_fmt = fmt if out_fmt is None else out_fmt
    m = Llama2(backend, config)
    shapes = config.matrix_shapes()
    for (name, l), val in weights.items():
        if name in LLAMA_MATRICES:
            r, c = shapes[name]
            m.set_matrix(name, l, GpuQuantMatrix(backend, fmt, r, c, val))
        elif name == "output":
            m.set_matrix(name, -1, GpuQuantMatrix(backend, out_fmt, config.vocab_size, config.dim, val))
        else:
            m.set_f32(name, l, val)
    return m


def synthetic_llama_device(backend: Backend, config: Llama2Config, fmt: int, out_fmt: int | None = None, seed: int = 0,
                           std: float = 0.02) -> Llama2:
    """Model-sized synthetic weights generated and quantised on the GPU (no host-side 7B-parameter arrays)."""
    out_fmt = fmt if out_fmt is None else out_fmt
    m = Llama2(backend, config)
    sid = seed * 1_000_003
    for l in range(config.n_layers):
        for i, (name, (r, c)) in enumerate(config.matrix_shapes().items()):
            m.set_matrix(name, l, GpuQuantMatrix.synthetic(backend, fmt, r, c, sid + 100 * l + i + 1, std))
        ones = np.ones(config.dim, dtype=np.float32)
        m.set_f32("attn_norm", l, ones)
        m.set_f32("ffn_norm", l, ones)
    emb = GpuVector(backend, config.vocab_size * config.dim)
    backend.check(backend.lib.slai_synth_normal_f32(backend.h, C.c_void_p(emb.ptr), emb.n, sid + 7_000_001, std))
    m.set_f32("token_embd", -1, emb)
    del emb
    m.set_f32("out_norm", -1, np.ones(config.dim, dtype=np.float32))
    m.set_matrix("output", -1, GpuQuantMatrix.synthetic(backend, out_fmt, config.vocab_size, config.dim, sid + 7_000_002, std))
    return m


# ---- GPT-2 ---------------------------------------------------------------------------------------------
@dataclass
class Gpt2Params:
    n_vocab: int
    n_seq: int
    n_embd: int
    n_head: int
    n_layer: int
    ff_len: int
    layernorm_eps: float = 1e-5
    kv_dtype: int = KV_F16

    def matrix_shapes(self):
        E = self.n_embd
        return dict(w_qkv=(3 * E, E), w_proj=(E, E), w_fc=(self.ff_len, E), w_fcproj=(E, self.ff_len))

    def weight_bytes_per_token(self, fmt: int) -> int:
        per = sum(r * c for r, c in self.matrix_shapes().values())
        bpw = synth.BITS_PER_WEIGHT[fmt]
        return int((self.n_layer * per + self.n_vocab * self.n_embd) * bpw / 8)


GPT2_XL = Gpt2Params(n_vocab=50257, n_seq=1024, n_embd=1600, n_head=25, n_layer=48, ff_len=6400)
GPT2_TINY = Gpt2Params(n_vocab=1031, n_seq=64, n_embd=128, n_head=4, n_layer=2, ff_len=512)


class Gpt2:
    def __init__(self, backend: Backend, params: Gpt2Params):
        self.backend, self.params = backend, params
        c = _CGpt2Config(params.n_vocab, params.n_seq, params.n_embd, params.n_head, params.n_layer, params.ff_len,
                         params.layernorm_eps, params.kv_dtype)
        h = C.c_void_p()
        backend.check(backend.lib.slai_gpt2_create(backend.h, C.byref(c), C.byref(h)))
        self.h = h
        self._keep = []

    def set_matrix(self, name: str, layer: int, m: GpuQuantMatrix):
        self._keep.append(m)
        self.backend.check(self.backend.lib.slai_gpt2_set_matrix(self.h, GPT2_W[name], layer, m.h))

    def set_f32(self, name: str, layer: int, data):
        a = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        self.backend.check(self.backend.lib.slai_gpt2_set_f32(self.h, GPT2_W[name], layer, a.ctypes.data_as(C.c_void_p), a.size))

    def forward(self, token: int, pos: int):
        logits = np.empty(self.params.n_vocab, dtype=np.float32)
        nxt = C.c_int32()
        self.backend.check(self.backend.lib.slai_gpt2_decode(self.h, token, pos, logits.ctypes.data_as(C.c_void_p), C.byref(nxt)))
        return logits, nxt.value

    def decode_into(self, token: int, pos: int, logits_ptr: int):
        nxt = C.c_int32()
        self.backend.check(self.backend.lib.slai_gpt2_decode(self.h, token, pos, C.c_void_p(logits_ptr), C.byref(nxt)))
        return nxt.value

    def generate(self, token: int, pos: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int32)
        self.backend.check(self.backend.lib.slai_gpt2_generate(self.h, token, pos, n, out.ctypes.data_as(C.c_void_p)))
        return out

    def prefill(self, tokens, pos0: int = 0, want_logits: bool = False):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.params.n_vocab, dtype=np.float32) if want_logits else None
        self.backend.check(self.backend.lib.slai_gpt2_prefill(self.h, t.ctypes.data_as(C.c_void_p), t.size, pos0,
                                                              logits.ctypes.data_as(C.c_void_p) if want_logits else None))
        return logits

    def close(self):
        if getattr(self, "h", None) and self.backend.h:
            self.backend.lib.slai_gpt2_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def synthetic_gpt2_host(p: Gpt2Params, fmt: int = synth.FMT_Q8_0, seed: int = 0, std: float = 0.02, bias_std: float = 0.0):
    """Seeded GPT-2 weights: gamma = 1, beta = 0, biases N(0, bias_std) (0 unless stated), wte quantised (tied)."""
    w = {}
    rng = np.random.default_rng(_seed(seed, "gpt2-bias", 0))
    E = p.n_embd
    for l in range(p.n_layer):
        for name, (r, c) in p.matrix_shapes().items():
            w[(name, l)] = synth.quantize(fmt, synth.normal_matrix(_seed(seed, name, l), r, c, std))
        for name, n in (("ln1_g", E), ("ln2_g", E)):
            w[(name, l)] = np.ones(n, dtype=np.float32)
        for name, n in (("ln1_b", E), ("ln2_b", E)):
            w[(name, l)] = np.zeros(n, dtype=np.float32)
        for name, n in (("b_qkv", 3 * E), ("b_proj", E), ("b_fc", p.ff_len), ("b_fcproj", E)):
            w[(name, l)] = (rng.standard_normal(n, dtype=np.float32) * np.float32(bias_std)).astype(np.float32)
    w[("wte", -1)] = synth.quantize(fmt, synth.normal_matrix(_seed(seed, "wte", -1), p.n_vocab, E, std))
    w[("wpe", -1)] = synth.normal_matrix(_seed(seed, "wpe", -1), p.n_seq, E, std)
    w[("lnf_g", -1)] = np.ones(E, dtype=np.float32)
    w[("lnf_b", -1)] = np.zeros(E, dtype=np.float32)
    return w


def gpt2_from_host(backend: Backend, p: Gpt2Params, weights: dict, fmt: int = synth.FMT_Q8_0) -> Gpt2:
    m = Gpt2(backend, p)
    shapes = p.matrix_shapes()
    for (name, l), val in weights.items():
        if name in GPT2_MATRICES:
            r, c = shapes[name]
            m.set_matrix(name, l, GpuQuantMatrix(backend, fmt, r, c, val))
        elif name == "wte":
            m.set_matrix(name, -1, GpuQuantMatrix(backend, fmt, p.n_vocab, p.n_embd, val))
        else:
            m.set_f32(name, l, val)
    return m


def synthetic_gpt2_device(backend: Backend, p: Gpt2Params, fmt: int = synth.FMT_Q8_0, seed: int = 0, std: float = 0.02) -> Gpt2:
    m = Gpt2(backend, p)
    sid = seed * 1_000_003 + 17
    E = p.n_embd
    for l in range(p.n_layer):
        for i, (name, (r, c)) in enumerate(p.matrix_shapes().items()):
            m.set_matrix(name, l, GpuQuantMatrix.synthetic(backend, fmt, r, c, sid + 100 * l + i + 1, std))
        m.set_f32("ln1_g", l, np.ones(E, np.float32)); m.set_f32("ln2_g", l, np.ones(E, np.float32))
        m.set_f32("ln1_b", l, np.zeros(E, np.float32)); m.set_f32("ln2_b", l, np.zeros(E, np.float32))
        m.set_f32("b_qkv", l, np.zeros(3 * E, np.float32)); m.set_f32("b_proj", l, np.zeros(E, np.float32))
        m.set_f32("b_fc", l, np.zeros(p.ff_len, np.float32)); m.set_f32("b_fcproj", l, np.zeros(E, np.float32))
    m.set_matrix("wte", -1, GpuQuantMatrix.synthetic(backend, fmt, p.n_vocab, E, sid + 7_000_001, std))
    m.set_f32("wpe", -1, synth.normal_matrix(_seed(seed, "wpe", -1), p.n_seq, E, std))
    m.set_f32("lnf_g", -1, np.ones(E, np.float32))
    m.set_f32("lnf_b", -1, np.zeros(E, np.float32))
    return m
