"""Synthetic GGUF-format inputs for the decode hot path (numpy, host side).

The reference tree contains no quantiser (its weights come from GGUF files), and no checkpoint is
available here, so tests and benchmarks build *valid* GGUF blocks from seeded normal floats with the
simple quantisers below.  Quantisation quality is irrelevant for parity: the CUDA path and the CPU
oracle consume exactly the same block bytes.  Block layouts follow
crates/slai/src/quantization.rs:29-32 (Q8_0), :204-209 (Q6_K), :249-255 (Q5_K), :322-327 (Q4_K) and
the 6-bit scale/min packing inverted from ``get_scale_min_k4`` (:381-389).

These are own-design quantisers (per-sub-block min/max), not ggml's.
"""
from __future__ import annotations

import numpy as np

FMT_F32, FMT_Q8_0, FMT_Q4_K, FMT_Q5_K, FMT_Q6_K = 0, 8, 12, 13, 14
# the legacy 32-element formats and Q8_K (crates/slai/src/quantization.rs:47-199): uploaded, not generated here
FMT_Q4_0, FMT_Q4_1, FMT_Q5_0, FMT_Q5_1, FMT_Q8_K = 2, 3, 6, 7, 15
LEGACY_FORMATS = (FMT_Q4_0, FMT_Q4_1, FMT_Q5_0, FMT_Q5_1, FMT_Q8_K)
FMT_NAMES = {FMT_F32: "f32", FMT_Q8_0: "q8_0", FMT_Q4_K: "q4_k", FMT_Q5_K: "q5_k", FMT_Q6_K: "q6_k", FMT_Q4_0: "q4_0", FMT_Q4_1: "q4_1",
             FMT_Q5_0: "q5_0", FMT_Q5_1: "q5_1", FMT_Q8_K: "q8_k"}
FMT_BY_NAME = {v: k for k, v in FMT_NAMES.items()}
BLOCK_BYTES = {FMT_F32: 4, FMT_Q8_0: 34, FMT_Q4_K: 144, FMT_Q5_K: 176, FMT_Q6_K: 210, FMT_Q4_0: 18, FMT_Q4_1: 20, FMT_Q5_0: 22, FMT_Q5_1: 24,
               FMT_Q8_K: 292}
BLOCK_ELEMS = {FMT_F32: 1, FMT_Q8_0: 32, FMT_Q4_K: 256, FMT_Q5_K: 256, FMT_Q6_K: 256, FMT_Q4_0: 32, FMT_Q4_1: 32, FMT_Q5_0: 32, FMT_Q5_1: 32,
               FMT_Q8_K: 256}
BITS_PER_WEIGHT = {FMT_F32: 32.0, FMT_Q8_0: 8.5, FMT_Q4_K: 4.5, FMT_Q5_K: 5.5, FMT_Q6_K: 6.5625, FMT_Q4_0: 4.5, FMT_Q4_1: 5.0, FMT_Q5_0: 5.5,
                   FMT_Q5_1: 6.0, FMT_Q8_K: 9.125}


def _f16_bits(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16).view(np.uint16)


def _f16_val(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16).astype(np.float32)


def _safe_div(a, b):
    return np.divide(a, b, out=np.zeros_like(a), where=b != 0)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """x: [..., K] f32, K % 32 == 0  ->  uint8 [..., K/32*34].  scale = absmax/127 as f16."""
    x = np.asarray(x, dtype=np.float32)
    lead, K = x.shape[:-1], x.shape[-1]
    assert K % 32 == 0
    b = x.reshape(-1, 32)
    scale = np.abs(b).max(axis=1) / np.float32(127.0)
    sv = _f16_val(scale)
    q = np.clip(np.rint(_safe_div(b, sv[:, None])), -127, 127).astype(np.int8)
    out = np.empty((b.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = _f16_bits(scale).reshape(-1, 1).view(np.uint8)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(*lead, K // 32 * 34)


def _pack_scales_k4(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """sc, m: [nb, 8] uint8 (6-bit) -> [nb, 12] bytes (inverse of get_scale_min_k4)."""
    out = np.empty((sc.shape[0], 12), dtype=np.uint8)
    out[:, 0:4] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = m[:, 0:4] | ((m[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0xF) | ((m[:, 4:8] & 0xF) << 4)
    return out


def _kquant_affine(x: np.ndarray, levels: int):
    """Shared part of Q4_K / Q5_K: returns (d_bits, dmin_bits, scales12, q[nb,256] uint8)."""
    b = x.reshape(-1, 8, 32)
    lo = np.minimum(b.min(axis=2), 0.0)
    hi = np.maximum(b.max(axis=2), lo)
    s = (hi - lo) / np.float32(levels)
    o = -lo
    d = s.max(axis=1) / np.float32(63.0)
    dmin = o.max(axis=1) / np.float32(63.0)
    dv, dminv = _f16_val(d), _f16_val(dmin)
    sc = np.clip(np.rint(_safe_div(s, dv[:, None])), 0, 63).astype(np.uint8)
    m = np.clip(np.rint(_safe_div(o, dminv[:, None])), 0, 63).astype(np.uint8)
    eff = dv[:, None] * sc.astype(np.float32)
    off = dminv[:, None] * m.astype(np.float32)
    q = np.clip(np.rint(_safe_div(b + off[:, :, None], eff[:, :, None])), 0, levels).astype(np.uint8)
    return _f16_bits(d), _f16_bits(dmin), _pack_scales_k4(sc, m), q.reshape(-1, 256)


def quantize_q4_k(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    lead, K = x.shape[:-1], x.shape[-1]
    assert K % 256 == 0
    d, dmin, scales, q = _kquant_affine(x, 15)
    nb = q.shape[0]
    out = np.empty((nb, 144), dtype=np.uint8)
    out[:, 0:2] = d.reshape(-1, 1).view(np.uint8)
    out[:, 2:4] = dmin.reshape(-1, 1).view(np.uint8)
    out[:, 4:16] = scales
    g = q.reshape(nb, 4, 2, 32)  # [group of 64][low/high half][l]
    out[:, 16:] = (g[:, :, 0, :] | (g[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(*lead, K // 256 * 144)


def quantize_q5_k(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    lead, K = x.shape[:-1], x.shape[-1]
    assert K % 256 == 0
    d, dmin, scales, q = _kquant_affine(x, 31)
    nb = q.shape[0]
    out = np.empty((nb, 176), dtype=np.uint8)
    out[:, 0:2] = d.reshape(-1, 1).view(np.uint8)
    out[:, 2:4] = dmin.reshape(-1, 1).view(np.uint8)
    out[:, 4:16] = scales
    g = q.reshape(nb, 4, 2, 32)
    qh = np.zeros((nb, 32), dtype=np.uint8)
    for G in range(4):
        qh |= ((g[:, G, 0, :] >> 4) & 1) << (2 * G)
        qh |= ((g[:, G, 1, :] >> 4) & 1) << (2 * G + 1)
    out[:, 16:48] = qh
    out[:, 48:] = ((g[:, :, 0, :] & 0xF) | ((g[:, :, 1, :] & 0xF) << 4)).reshape(nb, 128)
    return out.reshape(*lead, K // 256 * 176)


def quantize_q6_k(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    lead, K = x.shape[:-1], x.shape[-1]
    assert K % 256 == 0
    b = x.reshape(-1, 16, 16)
    s = np.abs(b).max(axis=2) / np.float32(32.0)
    d = s.max(axis=1) / np.float32(127.0)
    dv = _f16_val(d)
    sc = np.clip(np.rint(_safe_div(s, dv[:, None])), -128, 127).astype(np.int8)
    eff = dv[:, None] * sc.astype(np.float32)
    q = (np.clip(np.rint(_safe_div(b, eff[:, :, None])), -32, 31) + 32).astype(np.uint8).reshape(-1, 2, 4, 32)
    nb = q.shape[0]
    out = np.empty((nb, 210), dtype=np.uint8)
    ql = np.empty((nb, 2, 64), dtype=np.uint8)
    ql[:, :, 0:32] = (q[:, :, 0, :] & 0xF) | ((q[:, :, 2, :] & 0xF) << 4)
    ql[:, :, 32:64] = (q[:, :, 1, :] & 0xF) | ((q[:, :, 3, :] & 0xF) << 4)
    qh = (q[:, :, 0, :] >> 4) | ((q[:, :, 1, :] >> 4) << 2) | ((q[:, :, 2, :] >> 4) << 4) | ((q[:, :, 3, :] >> 4) << 6)
    out[:, 0:128] = ql.reshape(nb, 128)
    out[:, 128:192] = qh.reshape(nb, 64)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = _f16_bits(d).reshape(-1, 1).view(np.uint8)
    return out.reshape(*lead, K // 256 * 210)


def _pack_legacy(q: np.ndarray, bits: int, headers: list) -> np.ndarray:
    """q: [nb, 32] codes of `bits` (4 or 5) bits -> legacy block bytes: headers, [fifth bits,] 16 nibble bytes (element j
    in the low nibble of byte j, element j + 16 in the high nibble; fifth bit of element e is bit e of the 4-byte word)."""
    nb = q.shape[0]
    parts = [h.reshape(nb, -1) for h in headers]
    if bits == 5:
        word = np.zeros(nb, dtype=np.uint32)
        for e in range(32):
            word |= ((q[:, e].astype(np.uint32) >> 4) & 1) << e
        parts.append(word.reshape(nb, 1).view(np.uint8))
    lo = q & 0x0F
    parts.append((lo[:, :16] | (lo[:, 16:] << 4)).astype(np.uint8))
    return np.concatenate(parts, axis=1)


def quantize_legacy(fmt: int, x: np.ndarray) -> np.ndarray:
    """Simple own-design quantisers for the legacy formats (quantization.rs:47-199 defines the blocks, not how to fill them):
    Q4_0 / Q5_0 symmetric (d = absmax / 7 or / 15, code = round(x / d) + 8 or + 16), Q4_1 / Q5_1 affine (d = range / 15 or / 31,
    m = min), Q8_K d = absmax / 127 as f32."""
    x = np.asarray(x, dtype=np.float32)
    lead, K = x.shape[:-1], x.shape[-1]
    if fmt == FMT_Q8_K:
        b = x.reshape(-1, 256)
        d = (np.abs(b).max(axis=1) / np.float32(127.0)).astype(np.float32)
        q = np.clip(np.rint(_safe_div(b, d[:, None])), -127, 127).astype(np.int8)
        out = np.zeros((b.shape[0], 292), dtype=np.uint8)
        out[:, 0:4] = d.reshape(-1, 1).view(np.uint8)
        out[:, 4:260] = q.view(np.uint8)
        out[:, 260:] = q.reshape(-1, 16, 16).astype(np.int16).sum(axis=2).astype(np.int16).view(np.uint8).reshape(-1, 32)
        return out.reshape(*lead, K // 256 * 292)
    b = x.reshape(-1, 32)
    bits = 4 if fmt in (FMT_Q4_0, FMT_Q4_1) else 5
    top = (1 << bits) - 1
    if fmt in (FMT_Q4_0, FMT_Q5_0):
        half = 1 << (bits - 1)
        d = np.abs(b).max(axis=1) / np.float32(half - 1)
        dv = _f16_val(d)
        q = np.clip(np.rint(_safe_div(b, dv[:, None])) + half, 0, top).astype(np.uint8)
        out = _pack_legacy(q, bits, [_f16_bits(d).reshape(-1, 1).view(np.uint8)])
    else:
        lo, hi = b.min(axis=1), b.max(axis=1)
        d = (hi - lo) / np.float32(top)
        dv, mv = _f16_val(d), _f16_val(lo)
        q = np.clip(np.rint(_safe_div(b - mv[:, None], dv[:, None])), 0, top).astype(np.uint8)
        out = _pack_legacy(q, bits, [_f16_bits(d).reshape(-1, 1).view(np.uint8), _f16_bits(lo).reshape(-1, 1).view(np.uint8)])
    return out.reshape(*lead, K // 32 * BLOCK_BYTES[fmt])


_QUANTIZERS = {FMT_Q8_0: quantize_q8_0, FMT_Q4_K: quantize_q4_k, FMT_Q5_K: quantize_q5_k, FMT_Q6_K: quantize_q6_k,
               FMT_Q4_0: lambda x: quantize_legacy(FMT_Q4_0, x), FMT_Q4_1: lambda x: quantize_legacy(FMT_Q4_1, x),
               FMT_Q5_0: lambda x: quantize_legacy(FMT_Q5_0, x), FMT_Q5_1: lambda x: quantize_legacy(FMT_Q5_1, x),
               FMT_Q8_K: lambda x: quantize_legacy(FMT_Q8_K, x)}


def quantize(fmt: int, x: np.ndarray) -> np.ndarray:
    """Rows of f32 -> rows of GGUF block bytes (uint8 [M, K/elems*bytes])."""
    if fmt == FMT_F32:
        return np.ascontiguousarray(x, dtype=np.float32).view(np.uint8)
    return _QUANTIZERS[fmt](x)


def random_blocks(fmt: int, M: int, K: int, rng: np.random.Generator) -> np.ndarray:
    """Random bit patterns as blocks (the input style of the reference benchmark,
    crates/slai/src/ops/gemv_quant.rs:81-99) with the f16 super-block scales forced finite and small."""
    nbk = K // BLOCK_ELEMS[fmt]
    raw = rng.integers(0, 256, size=(M * nbk, BLOCK_BYTES[fmt]), dtype=np.uint8)
    d = _f16_bits(rng.uniform(1e-4, 2e-3, size=(M * nbk, 2)).astype(np.float32))
    if fmt == FMT_Q8_0:
        raw[:, 0:2] = d[:, 0:1].view(np.uint8)
    elif fmt in (FMT_Q4_K, FMT_Q5_K):
        raw[:, 0:4] = d.view(np.uint8).reshape(-1, 4)
    elif fmt == FMT_Q6_K:
        raw[:, 208:210] = d[:, 0:1].view(np.uint8)
    elif fmt in (FMT_Q4_0, FMT_Q5_0):
        raw[:, 0:2] = d[:, 0:1].view(np.uint8)
    elif fmt in (FMT_Q4_1, FMT_Q5_1):
        raw[:, 0:4] = d.view(np.uint8).reshape(-1, 4)
    elif fmt == FMT_Q8_K:
        raw[:, 0:4] = rng.uniform(1e-4, 2e-3, size=(M * nbk, 1)).astype(np.float32).view(np.uint8)
    return raw.reshape(M, nbk * BLOCK_BYTES[fmt])


def normal_matrix(seed, M: int, K: int, std: float = 0.02) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.standard_normal((M, K), dtype=np.float32) * np.float32(std)


def gemv_bytes(fmt: int, M: int, K: int) -> int:
    """Algorithmic HBM bytes of one quantised GEMV: packed weights + f32 input + f32 output."""
    return M * (K // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt] + 4 * K + 4 * M
