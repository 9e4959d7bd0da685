"""Host-side mirror of slai's operator interface for the decode path, on top of the C ABI.

Names, argument order and error behaviour follow the Rust operators (`crates/slai/src/ops/*.rs`) and the
dispatcher `LlmContext` (`crates/slai/src/context.rs`); each class cites the interface it stands for.
Tensors are plain device buffers (`GpuVector`) holding f32; nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
import enum

import numpy as np

from . import _lib
from ._lib import (AttnParams, SlaiError, FMT_F32, FMT_Q8_0, FMT_Q4_K, FMT_Q5_K, FMT_Q6_K, KV_F16, KV_F32)


class Backend:
    """The `B: Backend` of slang-hal as the decode path uses it: buffers, `write_buffer`, `read_buffer`,
    `synchronize` (call sites: crates/slai-chat/src/chat_llama2.rs:180-230).  One CUDA stream per backend."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        rc = self.lib.slai_ctx_create(device, C.byref(h))
        if rc != 0:
            raise SlaiError(rc, (self.lib.slai_last_error_string(None) or b"").decode() or "cannot create a context")
        self.h = h
        self.device = device

    # -- errors ------------------------------------------------------------------------------------
    def check(self, rc: int):
        if rc != 0:
            raise SlaiError(rc, (self.lib.slai_last_error_string(self.h) or b"").decode())

    # -- buffers -----------------------------------------------------------------------------------
    def malloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.check(self.lib.slai_malloc(self.h, nbytes, C.byref(p)))
        return p.value

    def free(self, ptr: int):
        if getattr(self, "_recording", False):
            self._deferred.append(ptr)  # a free would invalidate the recording (it synchronises the device)
            return
        self.check(self.lib.slai_free(self.h, C.c_void_p(ptr)))

    def write_buffer(self, dst: int, src: np.ndarray):
        src = np.ascontiguousarray(src)
        self.check(self.lib.slai_write_buffer(self.h, C.c_void_p(dst), src.ctypes.data_as(C.c_void_p), src.nbytes))
        self.synchronize()  # `src` may be a temporary

    def read_buffer(self, src: int, out: np.ndarray):
        assert out.flags["C_CONTIGUOUS"]
        self.check(self.lib.slai_read_buffer(self.h, out.ctypes.data_as(C.c_void_p), C.c_void_p(src), out.nbytes))
        return out

    def synchronize(self):
        self.check(self.lib.slai_ctx_sync(self.h))

    def vector(self, data, dtype=np.float32) -> "GpuVector":
        a = np.ascontiguousarray(data, dtype=dtype)
        v = GpuVector(self, a.size, dtype)
        self.write_buffer(v.ptr, a)
        return v

    def zeros(self, n: int, dtype=np.float32) -> "GpuVector":
        v = GpuVector(self, n, dtype)
        self.check(self.lib.slai_memset(self.h, C.c_void_p(v.ptr), 0, v.nbytes))
        return v

    def device_info(self):
        name = C.create_string_buffer(128)
        sms = C.c_int()
        self.check(self.lib.slai_ctx_device_info(self.h, name, 128, C.byref(sms)))
        return name.value.decode(), sms.value

    def mem_info(self):
        free, total = C.c_size_t(), C.c_size_t()
        self.check(self.lib.slai_ctx_mem_info(self.h, C.byref(free), C.byref(total)))
        return free.value, total.value

    def set_wait_limit(self, rounds: int):
        """Rounds a bounded device-side wait polls before it gives up (SLAI_ERR_TIMEOUT at the next synchronisation)."""
        self.check(self.lib.slai_ctx_set_wait_limit(self.h, rounds))

    def record(self) -> "RecordedPass":
        """Record the operator calls made inside the `with` block instead of running them (the reference's encoder:
        begin_pass ... submit, context.rs:63-96); replay with `.launch(times)`."""
        return RecordedPass(self)

    def timer_start(self):
        self.check(self.lib.slai_timer_start(self.h))

    def timer_stop(self) -> float:
        ms = C.c_float()
        self.check(self.lib.slai_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def close(self):
        if getattr(self, "h", None):
            self.lib.slai_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class RecordedPass:
    def __init__(self, backend: "Backend"):
        self.backend = backend
        self.h = C.c_void_p()

    def __enter__(self):
        self.backend._deferred = []
        self.backend._recording = True
        self.backend.check(self.backend.lib.slai_pass_begin(self.backend.h))
        return self

    def __exit__(self, et, ev, tb):
        rc = self.backend.lib.slai_pass_end(self.backend.h, C.byref(self.h))
        self.backend._recording = False
        for ptr in self.backend._deferred:  # buffers dropped by the garbage collector while recording
            self.backend.free(ptr)
        self.backend._deferred = []
        if et is None:
            self.backend.check(rc)
        return False

    def launch(self, times: int = 1):
        self.backend.check(self.backend.lib.slai_pass_launch(self.backend.h, self.h, times))

    def close(self):
        if self.h:
            self.backend.lib.slai_pass_destroy(self.backend.h, self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GpuVector:
    """`GpuVector<f32, B>` / `GpuTensor`: an owned device buffer (stensor, seen at context.rs:10-15)."""

    def __init__(self, backend: Backend, n: int, dtype=np.float32):
        self.backend = backend
        self.n = int(n)
        self.dtype = np.dtype(dtype)
        self.nbytes = self.n * self.dtype.itemsize
        self.ptr = backend.malloc(max(self.nbytes, 16))

    def __len__(self):
        return self.n

    def to_numpy(self) -> np.ndarray:
        out = np.empty(self.n, dtype=self.dtype)
        return self.backend.read_buffer(self.ptr, out)

    def view(self, offset: int, n: int) -> "GpuVectorView":
        assert 0 <= offset and offset + n <= self.n
        return GpuVectorView(self, offset, n)

    def __del__(self):
        try:
            if self.backend.h:
                self.backend.free(self.ptr)
        except Exception:
            pass


class GpuVectorView:
    """A contiguous sub-range of a `GpuVector` (`GpuTensorView`, e.g. `key_cache[l].column(pos)`)."""

    def __init__(self, base: GpuVector, offset: int, n: int):
        self.base, self.n = base, int(n)
        self.backend, self.dtype = base.backend, base.dtype
        self.ptr = base.ptr + offset * base.dtype.itemsize
        self.nbytes = self.n * base.dtype.itemsize

    def __len__(self):
        return self.n

    def to_numpy(self) -> np.ndarray:
        out = np.empty(self.n, dtype=self.dtype)
        return self.backend.read_buffer(self.ptr, out)


def _ptr(x) -> C.c_void_p:
    return C.c_void_p(x.ptr) if x is not None else C.c_void_p(None)


class GpuQuantMatrix:
    """`GpuQuantMatrix<B>` (crates/slai/src/quantized_matrix.rs:11-22) built like
    `GgufTensorData::to_gpu_matrix` (crates/slai/src/gguf.rs:133-194): raw GGUF blocks, row-major rows."""

    def __init__(self, backend: Backend, fmt: int, nrows: int, ncols: int, blocks: np.ndarray | None = None,
                 device_blocks: int | None = None, nbytes: int | None = None):
        self.backend = backend
        h = C.c_void_p()
        if blocks is not None:
            b = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
            self._keep = b
            backend.check(backend.lib.slai_qmatrix_create(backend.h, fmt, nrows, ncols, b.ctypes.data_as(C.c_void_p), b.size,
                                                          C.byref(h)))
        else:
            backend.check(backend.lib.slai_qmatrix_create_from_device(backend.h, fmt, nrows, ncols, C.c_void_p(device_blocks),
                                                                      nbytes, C.byref(h)))
        self.h = h
        self.fmt, self.nrows, self.ncols = fmt, nrows, ncols

    @classmethod
    def synthetic(cls, backend: Backend, fmt: int, nrows: int, ncols: int, seed: int, std: float, keep_raw: bool = False):
        """Blocks quantised on the device from seeded N(0, std) values (model-sized benchmark inputs)."""
        from .synth import BLOCK_BYTES, BLOCK_ELEMS
        nbytes = nrows * (ncols // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt]
        raw = GpuVector(backend, nbytes, np.uint8)
        backend.check(backend.lib.slai_synth_blocks(backend.h, fmt, nrows, ncols, seed, std, C.c_void_p(raw.ptr)))
        m = cls(backend, fmt, nrows, ncols, device_blocks=raw.ptr, nbytes=nbytes)
        backend.synchronize()
        if keep_raw:
            m.raw = raw
        return m

    def shape(self):
        return (self.nrows, self.ncols)

    def device_bytes(self) -> int:
        return int(self.backend.lib.slai_qmatrix_device_bytes(self.h))

    def dequantize(self) -> np.ndarray:
        """Bit-exact `Block*::dequantize()` of every block, evaluated on the device."""
        out = GpuVector(self.backend, self.nrows * self.ncols)
        self.backend.check(self.backend.lib.slai_qmatrix_dequantize(self.backend.h, self.h, C.c_void_p(out.ptr)))
        return out.to_numpy().reshape(self.nrows, self.ncols)

    def dequantize_row(self, row: int) -> np.ndarray:
        out = GpuVector(self.backend, self.ncols)
        self.backend.check(self.backend.lib.slai_qmatrix_dequantize_row(self.backend.h, self.h, row, C.c_void_p(out.ptr)))
        return out.to_numpy()

    def __del__(self):
        try:
            if self.backend.h and self.h and not getattr(self.backend, "_recording", False):
                self.backend.lib.slai_qmatrix_destroy(self.h)
                self.h = None
        except Exception:
            pass


class RoPEVariant(enum.IntEnum):
    """crates/slai/src/ops/rope.rs:8-14"""
    Original = 0
    Neox = 1


class UnaryOp(enum.IntEnum):
    """crates/slai/src/ops/unary.rs:11-35 (same order)"""
    Abs = 0
    Sgn = 1
    Neg = 2
    Step = 3
    Elu = 4
    Gelu = 5
    GeluQuick = 6
    Silu = 7
    Tanh = 8
    Sin = 9
    Cos = 10
    Relu = 11
    Sigmoid = 12
    HardSigmoid = 13
    Sqr = 14
    Sqrt = 15
    Log = 16
    LeakyRelu = 17
    Clamp = 18
    Scale = 19
    AddScalar = 20


class BatchedMultiqueryAttentionParams:
    """crates/slai/src/ops/batched_multiquery_attention.rs:17-29"""

    def __init__(self, seq_len, kv_dim, kv_mul, n_heads, head_size, pos):
        self.seq_len, self.kv_dim, self.kv_mul, self.n_heads, self.head_size, self.pos = seq_len, kv_dim, kv_mul, n_heads, head_size, pos

    def to_c(self) -> AttnParams:
        return AttnParams(self.seq_len, self.kv_dim, self.kv_mul, self.n_heads, self.head_size, self.pos)


class LlmContext:
    """`LlmContext<'a, B>` (crates/slai/src/context.rs:68-96): one method per operator; work is enqueued on the
    backend's stream (`begin_submission` ... `submit`), nothing blocks until `submit().synchronize()`."""

    def __init__(self, backend: Backend):
        self.backend = backend
        self.lib = backend.lib
        self.h = backend.h

    def begin_submission(self):  # context.rs:79-88 — recording is implicit: calls enqueue on the stream
        return self

    def submit(self):  # context.rs:90-95
        return self

    # GemvQuant::launch (ops/gemv_quant.rs:206-312); LlmContext::matmul_quant_assign (context.rs:355-369)
    def matmul_quant_assign(self, out, a: GpuQuantMatrix, b, n_batch: int = 1):
        if len(b) != a.ncols * n_batch or len(out) != a.nrows * n_batch:
            raise SlaiError(_lib.ERR_SHAPE, f"Gemv: dimension mismatch ({a.nrows}x{a.ncols} * {len(b)} -> {len(out)})")
        self.backend.check(self.lib.slai_gemv_quant(self.h, _ptr(out), a.h, _ptr(b), n_batch))

    def ffn_gate_up(self, out, w_gate: GpuQuantMatrix, w_up: GpuQuantMatrix, x, norm_w=None, eps: float = 1e-5):
        """out = silu(Wgate n(x)) * (Wup n(x)), n = RmsNorm: the operators of transformer.rs:356-361 as one kernel."""
        self.backend.check(self.lib.slai_ffn_gate_up(self.h, _ptr(out), w_gate.h, w_up.h, _ptr(x), _ptr(norm_w) if norm_w is not None else None, eps))

    # Tensor-parallel exchange operators (no counterpart in the reference): a row-parallel product whose partial goes
    # to every rank's exchange region, and a product whose input is the sum over ranks of such an exchange.
    def matmul_quant_partial(self, a: GpuQuantMatrix, b, resid, index: int, per_token: int):
        if len(b) != a.ncols or (resid is not None and len(resid) != a.nrows):
            raise SlaiError(_lib.ERR_SHAPE, "Gemv: dimension mismatch")
        self.backend.check(self.lib.slai_gemv_quant_partial(self.h, a.h, _ptr(b), _ptr(resid), index, per_token))

    def matmul_quant_reduced(self, out, a: GpuQuantMatrix, norm_w, eps: float, index: int, per_token: int, sum_out):
        if len(out) != a.nrows or len(norm_w) != a.ncols or len(sum_out) != a.ncols:
            raise SlaiError(_lib.ERR_SHAPE, "Gemv: dimension mismatch")
        self.backend.check(self.lib.slai_gemv_quant_reduced(self.h, _ptr(out), a.h, _ptr(norm_w), eps, index, per_token, _ptr(sum_out)))

    def token_tick(self):
        self.backend.check(self.lib.slai_tp_token_tick(self.h))

    def peer_loopback(self, ranks: int, rank: int):
        self.backend.check(self.lib.slai_tp_peer_loopback(self.h, ranks, rank))

    # RmsNorm::launch (ops/rms_norm.rs:35-67); LlmContext::rms_norm_assign
    def rms_norm_assign(self, result, value, weight, eps: float = 1e-5):
        if not (len(result) == len(value) == len(weight)):
            raise SlaiError(_lib.ERR_SHAPE, "rms_norm: length mismatch")
        self.backend.check(self.lib.slai_rms_norm(self.h, _ptr(result), _ptr(value), _ptr(weight), len(value), eps))

    # RoPE::launch (ops/rope.rs:45-85)
    def rope(self, variant: RoPEVariant, in_out_q, in_out_k, head_size: int, kv_dim: int, pos: int, base_freq: float = 10000.0):
        self.backend.check(self.lib.slai_rope(self.h, int(variant), _ptr(in_out_q), len(in_out_q), _ptr(in_out_k), head_size,
                                              kv_dim, pos, base_freq))

    # Silu::launch (ops/silu.rs:24-48)
    def silu(self, in_out_h1, in_h2):
        if len(in_out_h1) != len(in_h2):
            raise SlaiError(_lib.ERR_SHAPE, "silu: length mismatch")
        self.backend.check(self.lib.slai_silu_gate(self.h, _ptr(in_out_h1), _ptr(in_h2), len(in_out_h1)))

    # Unary::launch / launch_inplace (ops/unary.rs:171-306)
    def unary(self, op: UnaryOp, dest, src, args=(0.0, 0.0, 0.0, 0.0)):
        a = (C.c_float * 4)(*(list(args) + [0.0] * (4 - len(args))))
        self.backend.check(self.lib.slai_unary(self.h, int(op), _ptr(dest), _ptr(src), len(src), a))

    def gelu_inplace(self, x):
        self.unary(UnaryOp.Gelu, x, x)

    # SoftMax::launch_cols (ops/softmax.rs:22-40)
    def softmax_cols(self, in_out_mat, nrows: int, ncols: int, col_stride: int | None = None):
        self.backend.check(self.lib.slai_softmax_cols(self.h, _ptr(in_out_mat), nrows, ncols, col_stride or nrows))

    # LayerNorm::launch_cols (ops/layernorm.rs:25-60) (+ the caller's gamma/beta, gpt2/cpu.rs:239-240)
    def layernorm(self, output, input, eps: float = 1e-5, gamma=None, beta=None):
        if len(output) != len(input):
            raise SlaiError(_lib.ERR_SHAPE, "layernorm: length mismatch")
        self.backend.check(self.lib.slai_layernorm(self.h, _ptr(output), _ptr(input), len(input), eps, _ptr(gamma), _ptr(beta)))

    # LlmContext::add_assign / mul_assign / copy (context.rs:428-469,660-673)
    def add_assign(self, a, b):
        self.backend.check(self.lib.slai_add_assign(self.h, _ptr(a), _ptr(b), len(a)))

    def mul_assign(self, a, b):
        self.backend.check(self.lib.slai_mul_assign(self.h, _ptr(a), _ptr(b), len(a)))

    def copy(self, dst, src):
        self.backend.check(self.lib.slai_copy(self.h, _ptr(dst), _ptr(src), len(src)))

    # BatchedMultiqueryAttention::launch (ops/batched_multiquery_attention.rs:32-100)
    def attention(self, params: BatchedMultiqueryAttentionParams, q, key_cache, value_cache, xb, kv_dtype: int = KV_F32):
        p = params.to_c()
        self.backend.check(self.lib.slai_attention(self.h, C.byref(p), _ptr(q), _ptr(key_cache), _ptr(value_cache), kv_dtype, _ptr(xb)))

    def kv_append(self, key_cache, value_cache, k, v, kv_dim: int, pos: int, kv_dtype: int = KV_F32):
        self.backend.check(self.lib.slai_kv_append(self.h, _ptr(key_cache), _ptr(value_cache), kv_dtype, _ptr(k), _ptr(v), kv_dim, pos))

    def sample(self, logits: GpuVector, temperature: float, topp: float, coin: float) -> int:
        """`Sampler::sample` (models/sampler.rs:33-54) on the device, the uniform number `coin` given; `logits` is
        overwritten with the probabilities."""
        out = GpuVector(self.backend, 1, np.int32)
        self.backend.check(self.backend.lib.slai_sample(self.backend.h, C.c_void_p(logits.ptr), logits.n, temperature, topp, coin,
                                                        C.c_void_p(out.ptr)))
        return int(out.to_numpy()[0])

    # Sampler::sample_argmax (models/sampler.rs:55-57)
    def argmax(self, v) -> int:
        out = self.backend.zeros(1, np.int32)
        self.backend.check(self.lib.slai_argmax(self.h, _ptr(v), len(v), _ptr(out)))
        return int(out.to_numpy()[0])
