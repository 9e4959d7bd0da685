"""ctypes binding of libslai_b200.so (the C ABI declared in include/slai_b200.h).

There is no fallback: if the shared library is missing, or no sm_100 GPU is visible, every entry point of
the package raises.  Build the library with ``python -m slai_b200.build`` (or ``__graft_entry__.build()``).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SLAI_B200_LIB") or os.path.join(_HERE, "libslai_b200.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED_FORMAT, ERR_SHAPE, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_OOM = range(8)
STATUS_NAMES = ["OK", "INVALID_ARG", "UNSUPPORTED_FORMAT", "SHAPE", "CUDA", "NCCL", "TIMEOUT", "OOM"]

FMT_F32, FMT_F16, FMT_Q4_0, FMT_Q4_1, FMT_Q5_0, FMT_Q5_1, FMT_Q8_0 = 0, 1, 2, 3, 6, 7, 8
FMT_Q4_K, FMT_Q5_K, FMT_Q6_K, FMT_Q8_K = 12, 13, 14, 15
KV_F32, KV_F16 = 0, 1


class SlaiError(RuntimeError):
    """Mirror of the Rust wrapper's error enum: carries the C status code and the library's message."""

    def __init__(self, code: int, msg: str):
        self.code = code
        name = STATUS_NAMES[code] if 0 <= code < len(STATUS_NAMES) else str(code)
        super().__init__(f"slai_b200: {name}: {msg}")


class AttnParams(C.Structure):
    _fields_ = [("seq_len", C.c_uint32), ("kv_dim", C.c_uint32), ("kv_mul", C.c_uint32), ("n_heads", C.c_uint32),
                ("head_size", C.c_uint32), ("pos", C.c_uint32), ("_padding", C.c_uint32 * 2)]


class LlamaConfig(C.Structure):
    _fields_ = [("dim", C.c_int32), ("hidden_dim", C.c_int32), ("n_layers", C.c_int32), ("n_q_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("vocab_size", C.c_int32), ("seq_len", C.c_int32),
                ("rope_base_freq", C.c_float), ("rms_norm_eps", C.c_float), ("rope_variant", C.c_int32),
                ("kv_dtype", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32)]


class LlamaStats(C.Structure):
    """`slai_llama_stats_t`: microseconds and launches per kernel class of one decode step."""
    CLASSES = ("other", "qkv", "attention", "wo", "gate_up", "down", "logits")
    _fields_ = [("us_total", C.c_float), ("us", C.c_float * 7), ("launches", C.c_int32 * 7)]


class Gpt2Config(C.Structure):
    _fields_ = [("n_vocab", C.c_int32), ("n_seq", C.c_int32), ("n_embd", C.c_int32), ("n_head", C.c_int32),
                ("n_layer", C.c_int32), ("ff_len", C.c_int32), ("layernorm_eps", C.c_float), ("kv_dtype", C.c_int32)]


_vp, _i64, _i32, _sz, _f = C.c_void_p, C.c_int64, C.c_int32, C.c_size_t, C.c_float
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every function declared in include/slai_b200.h
SIGNATURES = {
    "slai_ctx_create": (C.c_int, [C.c_int, _pp]),
    "slai_ctx_destroy": (C.c_int, [_vp]),
    "slai_ctx_sync": (C.c_int, [_vp]),
    "slai_ctx_set_wait_limit": (C.c_int, [_vp, C.c_uint32]),
    "slai_tp_token_tick": (C.c_int, [_vp]),
    "slai_gemv_quant_partial": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int]),
    "slai_gemv_quant_reduced": (C.c_int, [_vp, _vp, _vp, _vp, _f, C.c_int, C.c_int, _vp]),
    "slai_tp_peer_loopback": (C.c_int, [_vp, C.c_int, C.c_int]),
    "slai_last_error_string": (C.c_char_p, [_vp]),
    "slai_ctx_stream": (_vp, [_vp]),
    "slai_device_count": (C.c_int, []),
    "slai_ctx_device_info": (C.c_int, [_vp, C.c_char_p, C.c_int, C.POINTER(C.c_int)]),
    "slai_ctx_mem_info": (C.c_int, [_vp, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "slai_malloc": (C.c_int, [_vp, _sz, _pp]),
    "slai_free": (C.c_int, [_vp, _vp]),
    "slai_memset": (C.c_int, [_vp, _vp, C.c_int, _sz]),
    "slai_write_buffer": (C.c_int, [_vp, _vp, _vp, _sz]),
    "slai_read_buffer": (C.c_int, [_vp, _vp, _vp, _sz]),
    "slai_malloc_host": (C.c_int, [_vp, _sz, _pp]),
    "slai_free_host": (C.c_int, [_vp, _vp]),
    "slai_pass_begin": (C.c_int, [_vp]),
    "slai_pass_end": (C.c_int, [_vp, _pp]),
    "slai_pass_launch": (C.c_int, [_vp, _vp, C.c_int]),
    "slai_pass_destroy": (C.c_int, [_vp, _vp]),
    "slai_tp_unique_id": (C.c_int, [_vp, _vp]),
    "slai_tp_init": (C.c_int, [_vp, _vp, C.c_int, C.c_int]),
    "slai_tp_all_reduce_sum": (C.c_int, [_vp, _vp, _vp, _i64]),
    "slai_tp_shutdown": (C.c_int, [_vp]),
    "slai_tp_peer_export": (C.c_int, [_vp, _vp]),
    "slai_tp_peer_attach": (C.c_int, [_vp, _vp]),
    "slai_timer_start": (C.c_int, [_vp]),
    "slai_timer_stop": (C.c_int, [_vp, C.POINTER(_f)]),
    "slai_qmatrix_create": (C.c_int, [_vp, C.c_int, _i64, _i64, _vp, _sz, _pp]),
    "slai_qmatrix_create_from_device": (C.c_int, [_vp, C.c_int, _i64, _i64, _vp, _sz, _pp]),
    "slai_qmatrix_destroy": (C.c_int, [_vp]),
    "slai_qmatrix_shape": (C.c_int, [_vp, C.POINTER(C.c_int), C.POINTER(_i64), C.POINTER(_i64)]),
    "slai_qmatrix_device_bytes": (_sz, [_vp]),
    "slai_qmatrix_dequantize": (C.c_int, [_vp, _vp, _vp]),
    "slai_qmatrix_dequantize_row": (C.c_int, [_vp, _vp, _i64, _vp]),
    "slai_synth_blocks": (C.c_int, [_vp, C.c_int, _i64, _i64, C.c_uint64, _f, _vp]),
    "slai_synth_normal_f32": (C.c_int, [_vp, _vp, _i64, C.c_uint64, _f]),
    "slai_gemv_quant": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int]),
    "slai_ffn_gate_up": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _f]),
    "slai_rms_norm": (C.c_int, [_vp, _vp, _vp, _vp, _i64, _f]),
    "slai_rope": (C.c_int, [_vp, C.c_int, _vp, _i64, _vp, C.c_int, C.c_int, C.c_int, _f]),
    "slai_silu_gate": (C.c_int, [_vp, _vp, _vp, _i64]),
    "slai_unary": (C.c_int, [_vp, C.c_int, _vp, _vp, _i64, C.POINTER(_f)]),
    "slai_softmax_cols": (C.c_int, [_vp, _vp, _i64, _i64, _i64]),
    "slai_layernorm": (C.c_int, [_vp, _vp, _vp, _i64, _f, _vp, _vp]),
    "slai_add_assign": (C.c_int, [_vp, _vp, _vp, _i64]),
    "slai_mul_assign": (C.c_int, [_vp, _vp, _vp, _i64]),
    "slai_copy": (C.c_int, [_vp, _vp, _vp, _i64]),
    "slai_argmax": (C.c_int, [_vp, _vp, _i64, _vp]),
    "slai_attention": (C.c_int, [_vp, C.POINTER(AttnParams), _vp, _vp, _vp, C.c_int, _vp]),
    "slai_attention_static": (C.c_int, [_vp, C.POINTER(AttnParams), _vp, _vp, _vp, C.c_int, _vp]),
    "slai_kv_append": (C.c_int, [_vp, _vp, _vp, C.c_int, _vp, _vp, C.c_int, C.c_int]),
    "slai_llama_create": (C.c_int, [_vp, C.POINTER(LlamaConfig), _pp]),
    "slai_llama_destroy": (C.c_int, [_vp]),
    "slai_llama_set_matrix": (C.c_int, [_vp, C.c_int, C.c_int, _vp]),
    "slai_llama_set_f32": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _i64]),
    "slai_llama_set_f32_device": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _i64]),
    "slai_llama_decode": (C.c_int, [_vp, _i32, _i32, _vp, C.POINTER(_i32)]),
    "slai_llama_generate": (C.c_int, [_vp, _i32, _i32, _i32, _vp]),
    "slai_llama_generate_sampled": (C.c_int, [_vp, _i32, _i32, _i32, C.c_float, C.c_float, C.c_uint64, _vp]),
    "slai_sample": (C.c_int, [_vp, _vp, _i64, C.c_float, C.c_float, C.c_float, _vp]),
    "slai_llama_prefill": (C.c_int, [_vp, _vp, _i32, _i32, _vp]),
    "slai_llama_read_kv": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _vp]),
    "slai_llama_stats": (C.c_int, [_vp, C.c_int32, C.c_int32, _vp]),
    "slai_llama_batch_reserve": (C.c_int, [_vp, _i32]),
    "slai_llama_decode_batch": (C.c_int, [_vp, _i32, _vp, _vp, _vp, _vp]),
    "slai_llama_read_state": (C.c_int, [_vp, C.c_int, _vp, _i64]),
    "slai_llama_launches_per_token": (C.c_int, [_vp]),
    "slai_gpt2_create": (C.c_int, [_vp, C.POINTER(Gpt2Config), _pp]),
    "slai_gpt2_destroy": (C.c_int, [_vp]),
    "slai_gpt2_set_matrix": (C.c_int, [_vp, C.c_int, C.c_int, _vp]),
    "slai_gpt2_set_f32": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _i64]),
    "slai_gpt2_decode": (C.c_int, [_vp, _i32, _i32, _vp, C.POINTER(_i32)]),
    "slai_gpt2_generate": (C.c_int, [_vp, _i32, _i32, _i32, _vp]),
    "slai_gpt2_prefill": (C.c_int, [_vp, _vp, _i32, _i32, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library.  Raises if it has not been built: there is no CPU path to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SlaiError(ERR_CUDA, f"{LIB_PATH} is missing: build it with `python -m slai_b200.build` "
                                      "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
