"""ctypes binding of the CPU oracle (TEST INFRASTRUCTURE, not part of the product).

Only the tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` import this
module.  It loads ``libslai_oracle.so`` (built by ``make -C oracle``) which restates the CPU
operator path of dimforge/slai; see the header of ``slai_oracle.cpp`` for what pins it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libslai_oracle.so")

FMT_F32, FMT_Q8_0, FMT_Q4_K, FMT_Q5_K, FMT_Q6_K = 0, 8, 12, 13, 14

UNARY_OPS = [
    "abs", "sgn", "neg", "step", "elu", "gelu", "gelu_quick", "silu", "tanh", "sin", "cos", "relu",
    "sigmoid", "hard_sigmoid", "sqr", "sqrt", "log", "leaky_relu", "clamp", "scale", "add_scalar",
]

# weight ids (same numbering as include/slai_b200.h)
LLAMA_W = dict(token_embd=0, out_norm=1, output=2, attn_norm=3, wq=4, wk=5, wv=6, wo=7, ffn_norm=8,
               w_gate=9, w_up=10, w_down=11, bq=12, bk=13, bv=14)
GPT2_W = dict(wte=0, wpe=1, lnf_g=2, lnf_b=3, ln1_g=4, ln1_b=5, w_qkv=6, b_qkv=7, w_proj=8, b_proj=9,
              ln2_g=10, ln2_b=11, w_fc=12, b_fc=13, w_fcproj=14, b_fcproj=15)


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "slai_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libslai_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        f32p, vp, i64 = C.POINTER(C.c_float), C.c_void_p, C.c_int64
        L.ora_decode_f16.restype = C.c_float
        L.ora_decode_f16.argtypes = [C.c_uint16]
        L.ora_encode_f16.restype = C.c_uint16
        L.ora_encode_f16.argtypes = [C.c_float]
        L.ora_dequantize.argtypes = [C.c_int, vp, i64, vp]
        L.ora_gemv_f32.argtypes = [vp, vp, vp, i64, i64, C.c_int]
        L.ora_gemv_f64acc.argtypes = [vp, vp, vp, i64, i64]
        L.ora_gemv_quant.argtypes = [C.c_int, vp, vp, vp, i64, i64, C.c_int]
        L.ora_rms_norm.argtypes = [vp, vp, vp, i64, C.c_float]
        L.ora_layernorm.argtypes = [vp, vp, i64, C.c_float]
        L.ora_softmax.argtypes = [vp, i64]
        L.ora_silu_gate.argtypes = [vp, vp, i64]
        L.ora_unary.argtypes = [C.c_int, vp, vp, i64, vp]
        L.ora_rope.argtypes = [C.c_int, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        L.ora_attention.argtypes = [C.c_int] * 6 + [vp] * 5
        L.ora_argmax.argtypes = [vp, i64]
        L.ora_llama_create.restype = vp
        L.ora_llama_create.argtypes = [C.c_int] * 7 + [C.c_float, C.c_float, C.c_int, C.c_int, C.c_int]
        L.ora_llama_destroy.argtypes = [vp]
        L.ora_llama_set_weight.argtypes = [vp, C.c_int, C.c_int, vp]
        L.ora_llama_forward.restype = f32p
        L.ora_llama_forward.argtypes = [vp, C.c_int, C.c_int]
        L.ora_llama_x.restype = f32p
        L.ora_llama_x.argtypes = [vp]
        L.ora_gpt2_create.restype = vp
        L.ora_gpt2_create.argtypes = [C.c_int] * 6 + [C.c_float, C.c_int, C.c_int]
        L.ora_gpt2_destroy.argtypes = [vp]
        L.ora_gpt2_set_weight.argtypes = [vp, C.c_int, C.c_int, vp]
        L.ora_gpt2_forward.restype = f32p
        L.ora_gpt2_forward.argtypes = [vp, C.c_int, C.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


BLOCK_BYTES = {FMT_F32: 4, FMT_Q8_0: 34, FMT_Q4_K: 144, FMT_Q5_K: 176, FMT_Q6_K: 210, 2: 18, 3: 20, 6: 22, 7: 24, 15: 292}
BLOCK_ELEMS = {FMT_F32: 1, FMT_Q8_0: 32, FMT_Q4_K: 256, FMT_Q5_K: 256, FMT_Q6_K: 256, 2: 32, 3: 32, 6: 32, 7: 32, 15: 256}


def decode_f16(h: int) -> float:
    return float(lib().ora_decode_f16(int(h)))


def encode_f16(x: float) -> int:
    return int(lib().ora_encode_f16(float(x)))


def dequantize(fmt: int, blocks: np.ndarray) -> np.ndarray:
    """Raw GGUF block bytes (uint8) -> f32 values in element order."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    nb = blocks.size // BLOCK_BYTES[fmt]
    assert nb * BLOCK_BYTES[fmt] == blocks.size
    out = np.empty(nb * BLOCK_ELEMS[fmt], dtype=np.float32)
    rc = lib().ora_dequantize(fmt, _p(blocks), nb, _p(out))
    assert rc == 0
    return out


def gemv_f32(w: np.ndarray, x: np.ndarray, nthreads: int = 1) -> np.ndarray:
    w, x = _f32(w), _f32(x)
    M, K = w.shape
    out = np.empty(M, dtype=np.float32)
    lib().ora_gemv_f32(_p(out), _p(w), _p(x), M, K, nthreads)
    return out


def gemv_f64acc(w: np.ndarray, x: np.ndarray) -> np.ndarray:
    w, x = _f32(w), _f32(x)
    M, K = w.shape
    out = np.empty(M, dtype=np.float32)
    lib().ora_gemv_f64acc(_p(out), _p(w), _p(x), M, K)
    return out


def gemv_quant(fmt: int, blocks: np.ndarray, x: np.ndarray, M: int, K: int, nthreads: int = 1) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    x = _f32(x)
    out = np.empty(M, dtype=np.float32)
    rc = lib().ora_gemv_quant(fmt, _p(out), _p(blocks), _p(x), M, K, nthreads)
    assert rc == 0
    return out


def rms_norm(a, w, eps: float = 1e-5) -> np.ndarray:
    a, w = _f32(a), _f32(w)
    out = np.empty_like(a)
    lib().ora_rms_norm(_p(out), _p(a), _p(w), a.size, eps)
    return out


def layernorm(v, eps: float = 1e-5) -> np.ndarray:
    v = _f32(v)
    out = np.empty_like(v)
    lib().ora_layernorm(_p(out), _p(v), v.size, eps)
    return out


def softmax(v) -> np.ndarray:
    out = _f32(v).copy()
    lib().ora_softmax(_p(out), out.size)
    return out


def silu_gate(h1, h2) -> np.ndarray:
    out, h2 = _f32(h1).copy(), _f32(h2)
    lib().ora_silu_gate(_p(out), _p(h2), out.size)
    return out


def unary(op: str | int, x, args=(0.0, 0.0, 0.0, 0.0)) -> np.ndarray:
    opi = UNARY_OPS.index(op) if isinstance(op, str) else int(op)
    x = _f32(x)
    out = np.empty_like(x)
    a = np.asarray(list(args) + [0.0] * (4 - len(args)), dtype=np.float32)
    lib().ora_unary(opi, _p(out), _p(x), x.size, _p(a))
    return out


def rope(q, k, head_size: int, kv_dim: int, pos: int, base: float = 10000.0, neox: bool = False):
    q, k = _f32(q).copy(), _f32(k).copy()
    lib().ora_rope(int(neox), _p(q), _p(k), head_size, q.size, kv_dim, pos, base)
    return q, k


def attention(q, key_cache, value_cache, *, seq_len, kv_dim, kv_mul, n_heads, head_size, pos):
    """key_cache/value_cache: [seq_len, kv_dim] f32 (position-major)."""
    q, kc, vc = _f32(q), _f32(key_cache), _f32(value_cache)
    att = np.zeros((n_heads, seq_len), dtype=np.float32)
    xb = np.empty(n_heads * head_size, dtype=np.float32)
    lib().ora_attention(seq_len, kv_dim, kv_mul, n_heads, head_size, pos, _p(q), _p(kc), _p(vc), _p(att), _p(xb))
    return xb, att


def sample(logits, temperature: float, topp: float, coin: float):
    """`Sampler::sample` with the random draw `coin` given; returns (token id, probabilities)."""
    p = _f32(logits).copy()
    lib().ora_sample.restype = C.c_int
    lib().ora_sample.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_float, C.c_float]
    return int(lib().ora_sample(_p(p), p.size, temperature, topp, coin)), p


def argmax(v) -> int:
    v = _f32(v)
    return int(lib().ora_argmax(_p(v), v.size))


class Llama:
    """Dense-f32 CPU twin of ``llama2::cpu::Transformer``; weights are dequantised by the caller."""

    def __init__(self, *, dim, hidden, n_layers, n_q, n_kv, vocab, seq_len, rope_base=10000.0, eps=1e-5,
                 neox=False, kv_f16=False, nthreads=1):
        self.cfg = dict(dim=dim, hidden=hidden, n_layers=n_layers, n_q=n_q, n_kv=n_kv, vocab=vocab, seq_len=seq_len)
        self._h = lib().ora_llama_create(dim, hidden, n_layers, n_q, n_kv, vocab, seq_len, rope_base, eps,
                                         int(neox), int(kv_f16), nthreads)
        self._keep = []

    def set_weight(self, name: str, layer: int, arr: np.ndarray):
        arr = _f32(arr)
        self._keep.append(arr)
        rc = lib().ora_llama_set_weight(self._h, LLAMA_W[name], layer, _p(arr))
        assert rc == 0, name

    def forward(self, token: int, pos: int) -> np.ndarray:
        p = lib().ora_llama_forward(self._h, int(token), int(pos))
        return np.ctypeslib.as_array(p, shape=(self.cfg["vocab"],)).copy()

    def x(self) -> np.ndarray:
        return np.ctypeslib.as_array(lib().ora_llama_x(self._h), shape=(self.cfg["dim"],)).copy()

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ora_llama_destroy(self._h)
            self._h = None


class Gpt2:
    """Dense-f32 CPU twin of ``gpt2::cpu::Transformer``."""

    def __init__(self, *, n_vocab, n_seq, n_embd, n_head, n_layer, ff_len, eps=1e-5, kv_f16=False, nthreads=1):
        self.cfg = dict(n_vocab=n_vocab, n_seq=n_seq, n_embd=n_embd, n_head=n_head, n_layer=n_layer, ff_len=ff_len)
        self._h = lib().ora_gpt2_create(n_vocab, n_seq, n_embd, n_head, n_layer, ff_len, eps, int(kv_f16), nthreads)
        self._keep = []

    def set_weight(self, name: str, layer: int, arr: np.ndarray):
        arr = _f32(arr)
        self._keep.append(arr)
        rc = lib().ora_gpt2_set_weight(self._h, GPT2_W[name], layer, _p(arr))
        assert rc == 0, name

    def forward(self, token: int, pos: int) -> np.ndarray:
        p = lib().ora_gpt2_forward(self._h, int(token), int(pos))
        return np.ctypeslib.as_array(p, shape=(self.cfg["n_vocab"],)).copy()

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ora_gpt2_destroy(self._h)
            self._h = None
