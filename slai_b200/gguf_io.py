"""GGUF files -> models on the GPU (the reference's `Gguf::from_bytes` + `Llama2Config::from_gguf` +
`Llama2Weights::from_gguf`: crates/slai/src/gguf.rs:503-679, models/llama2/cpu.rs:76-108,
models/llama2/transformer.rs:201-297).

A small reader written from the published GGUF layout (versions 2 and 3, little endian):

    magic "GGUF" | u32 version | u64 n_tensors | u64 n_kv
    n_kv     x { string key, u32 value type, value }          string = u64 length + bytes; arrays = u32 type, u64 count, items
    n_tensors x { string name, u32 n_dims, u64 dims[n_dims], u32 ggml type, u64 offset }
    padding to `general.alignment` (default 32), then the tensor data; offsets are relative to that point.

dims[0] is the contiguous (column) dimension.  Quantised tensors are handed to the library as the file's bytes
(memory-mapped, no conversion): `slai_qmatrix_create` re-tiles them on the device.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np

from . import synth
from ._lib import KV_F16
from .models import Llama2, Llama2Config
from .ops import Backend, GpuQuantMatrix

GGUF_MAGIC = b"GGUF"
# ggml type id -> (elements per block, bytes per block)
GGML_BLOCK = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 36), 10: (256, 84),
              11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292), 30: (1, 2)}
GGML_F32, GGML_F16 = 0, 1
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


class GgufError(ValueError):
    pass


@dataclass
class GgufTensor:
    name: str
    dims: tuple          # as stored: dims[0] = columns
    ggml_type: int
    data: np.ndarray     # uint8 view of the file's bytes for this tensor

    @property
    def cols(self) -> int:
        return int(self.dims[0])

    @property
    def rows(self) -> int:
        n = 1
        for d in self.dims[1:]:
            n *= int(d)
        return n

    def to_f32(self) -> np.ndarray:
        if self.ggml_type == GGML_F32:
            return self.data.view(np.float32).copy()
        if self.ggml_type == GGML_F16:
            return self.data.view(np.float16).astype(np.float32)
        raise GgufError(f"{self.name}: type {self.ggml_type} is not a plain float tensor")


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError("truncated file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufError("truncated string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype: int):
        if vtype in _SCALAR:
            return self.take(_SCALAR[vtype])
        if vtype == _T_STRING:
            return self.string()
        if vtype == _T_ARRAY:
            itype = self.take("<I")
            count = self.take("<Q")
            if itype in _SCALAR and itype != 7:
                size = struct.calcsize(_SCALAR[itype])
                if self.pos + size * count > len(self.buf):
                    raise GgufError("truncated array")
                arr = np.frombuffer(self.buf, dtype=np.dtype(_SCALAR[itype][1:]).newbyteorder("<"), count=count, offset=self.pos)
                self.pos += size * count
                return arr
            return [self.value(itype) for _ in range(count)]
        raise GgufError(f"unknown metadata value type {vtype}")


class GgufFile:
    """Parsed header of a GGUF file; tensor bytes stay memory-mapped."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        buf = memoryview(self._map)
        c = _Cursor(buf)
        if bytes(buf[:4]) != GGUF_MAGIC:
            raise GgufError("not a GGUF file")
        c.pos = 4
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise GgufError(f"GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        self.metadata: dict = {}
        for _ in range(n_kv):
            key = c.string()
            self.metadata[key] = c.value(c.take("<I"))
        infos = []
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            dims = tuple(c.take("<Q") for _ in range(nd))
            infos.append((name, dims, c.take("<I"), c.take("<Q")))
        align = int(self.metadata.get("general.alignment", 32))
        base = (c.pos + align - 1) // align * align
        whole = np.frombuffer(buf, dtype=np.uint8)
        self.tensors: dict[str, GgufTensor] = {}
        for name, dims, gt, off in infos:
            if gt not in GGML_BLOCK:
                raise GgufError(f"{name}: unknown ggml type {gt}")
            be, bb = GGML_BLOCK[gt]
            n = 1
            for d in dims:
                n *= int(d)
            if dims and int(dims[0]) % be:
                raise GgufError(f"{name}: row length {dims[0]} is not a multiple of the block size {be}")
            nbytes = n // be * bb
            if base + off + nbytes > len(whole):
                raise GgufError(f"{name}: data runs past the end of the file")
            self.tensors[name] = GgufTensor(name, dims, gt, whole[base + off:base + off + nbytes])

    def close(self):
        self.tensors = {}
        try:
            self._map.close()
        except BufferError:
            pass  # numpy views still alive: the map goes with them
        self._f.close()


def llama_config_from_gguf(g: GgufFile, model_name: str = "llama", kv_dtype: int = KV_F16) -> Llama2Config:
    """Same keys and defaults as Llama2Config::from_gguf_with_model_type (models/llama2/cpu.rs:79-108)."""
    md = g.metadata

    def need(key):
        if key not in md:
            raise GgufError(f"metadata key {key} is missing")
        return md[key]

    return Llama2Config(dim=int(need(f"{model_name}.embedding_length")), hidden_dim=int(need(f"{model_name}.feed_forward_length")),
                        n_layers=int(need(f"{model_name}.block_count")), n_q_heads=int(need(f"{model_name}.attention.head_count")),
                        n_kv_heads=int(need(f"{model_name}.attention.head_count_kv")), vocab_size=len(need("tokenizer.ggml.tokens")),
                        seq_len=int(need(f"{model_name}.context_length")), rope_base_freq=float(md.get(f"{model_name}.rope.freq_base", 10000.0)),
                        rms_norm_eps=float(md.get(f"{model_name}.attention.layer_norm_rms_epsilon", 1.0e-6)), kv_dtype=kv_dtype)


_LAYER_TENSORS = dict(wq="attn_q.weight", wk="attn_k.weight", wv="attn_v.weight", wo="attn_output.weight", w_gate="ffn_gate.weight",
                      w_up="ffn_up.weight", w_down="ffn_down.weight")
_LAYER_VECTORS = dict(attn_norm="attn_norm.weight", ffn_norm="ffn_norm.weight", bq="attn_q.bias", bk="attn_k.bias", bv="attn_v.bias")
_QUANT_OK = (synth.FMT_Q8_0, synth.FMT_Q4_K, synth.FMT_Q5_K, synth.FMT_Q6_K)


def _matrix(backend: Backend, t: GgufTensor) -> GpuQuantMatrix:
    """GgufTensor::to_gpu_matrix (gguf.rs:357-366): quantised tensors stay quantised, float tensors become f32."""
    if t.ggml_type in _QUANT_OK:
        return GpuQuantMatrix(backend, t.ggml_type, t.rows, t.cols, t.data)
    if t.ggml_type in (GGML_F32, GGML_F16):
        return GpuQuantMatrix(backend, synth.FMT_F32, t.rows, t.cols, t.to_f32().view(np.uint8))
    raise GgufError(f"{t.name}: ggml type {t.ggml_type} has no kernel (supported: F32, F16, Q8_0, Q4_K, Q5_K, Q6_K)")


def llama_from_gguf(backend: Backend, g: GgufFile, model_name: str = "llama", kv_dtype: int = KV_F16) -> Llama2:
    """Llama2Weights::from_gguf (models/llama2/transformer.rs:201-297): tensor names `blk.{i}.attn_q.weight` ...,
    `token_embd.weight`, `output_norm.weight`, optional `output.weight` (absent: tied to the embedding)."""
    cfg = llama_config_from_gguf(g, model_name, kv_dtype)
    m = Llama2(backend, cfg)
    for l in range(cfg.n_layers):
        for ours, theirs in _LAYER_TENSORS.items():
            name = f"blk.{l}.{theirs}"
            if name not in g.tensors:
                raise GgufError(f"tensor {name} is missing")
            m.set_matrix(ours, l, _matrix(backend, g.tensors[name]))
        for ours, theirs in _LAYER_VECTORS.items():
            name = f"blk.{l}.{theirs}"
            if name in g.tensors:
                m.set_f32(ours, l, g.tensors[name].to_f32())
            elif ours in ("attn_norm", "ffn_norm"):
                raise GgufError(f"tensor {name} is missing")
    emb = g.tensors.get("token_embd.weight")
    if emb is None:
        raise GgufError("tensor token_embd.weight is missing")
    if emb.ggml_type in (GGML_F32, GGML_F16):
        m.set_f32("token_embd", -1, emb.to_f32())
    elif emb.ggml_type == synth.FMT_Q8_0:
        m.set_matrix("token_embd", -1, _matrix(backend, emb))
    else:  # K-quant embedding table: dequantised once on the device (rows are looked up, not multiplied)
        m.set_f32("token_embd", -1, _matrix(backend, emb).dequantize())
    m.set_f32("out_norm", -1, g.tensors["output_norm.weight"].to_f32())
    if "output.weight" in g.tensors:
        m.set_matrix("output", -1, _matrix(backend, g.tensors["output.weight"]))
    return m
