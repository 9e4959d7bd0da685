"""Second description of the decode operators' arithmetic, taken from the reference's GPU shaders.

TEST INFRASTRUCTURE ONLY.  The oracle (oracle/slai_oracle.cpp) restates the reference's CPU operator path; the
functions here restate, in numpy and in this repository's own words, what the reference's Slang compute shaders
do for the same operators: which lane of a 32-thread group dequantises which element with which scale, in which
order partial sums meet.  The two descriptions come from different source files of the reference
(crates/slai/src/*.rs on one side, crates/slai/shaders/slai/*.slang on the other); tests/test_shader_pin.py
requires them to agree: dequantised values bit for bit, sums within the rounding of their different summation
orders.  Nothing is compiled from the shaders and the product never imports this module.

All arithmetic is float32 with one rounding per operation (no fused multiply-add), like the oracle's build.
"""
from __future__ import annotations

import numpy as np

f32 = np.float32


def _words(block_bytes: np.ndarray) -> np.ndarray:
    """A block as the little-endian u32 words the shaders index (StructuredBuffer<uint>)."""
    return np.frombuffer(np.ascontiguousarray(block_bytes).tobytes(), dtype="<u4")


def _half_lo(word):  # unpackHalf2x16ToHalf(word).x
    return np.array([int(word) & 0xFFFF], dtype=np.uint16).view(np.float16).astype(f32)[0]


def _half_hi(word):  # .y
    return np.array([(int(word) >> 16) & 0xFFFF], dtype=np.uint16).view(np.float16).astype(f32)[0]


def _i8x4(word):  # unpackInt4x8ToInt32
    return np.array([int(word) & 0xFFFFFFFF], dtype="<u4").view(np.int8).astype(np.int32)


def _u8x4(word):  # unpackUint4x8ToUint32
    return np.array([int(word) & 0xFFFFFFFF], dtype="<u4").view(np.uint8).astype(np.uint32)


def _scale_min_6bit(j, prev, cur, nxt):
    """BlockQ4K.unpack_scale_and_min (gemv_quant_q4_k.slang:79-94): 6-bit scale and minimum of sub-block j from the
    three words around it."""
    sh = (j % 4) * 8
    p, c, n = (int(prev) >> sh) & 0xFF, (int(cur) >> sh) & 0xFF, (int(nxt) >> sh) & 0xFF
    if j < 4:
        return c & 63, n & 63
    return (n & 0xF) | ((p >> 6) << 4), (n >> 4) | ((c >> 6) << 4)


# ---------------------------------------------------------------------------------------------------------
# Lane -> element maps.  Each returns, for ONE block (or block pair) and lane k of the 32-thread group, a list of
# (first element index inside the block (pair), four dequantised f32 values).
# ---------------------------------------------------------------------------------------------------------
def q4k_lane(w: np.ndarray, k: int, five: bool = False):
    """gemv_quant_q4_k.slang:96-147 (Q4_K, 36 words) / gemv_quant_q5_k.slang:82-130 (Q5_K, 44 words).
    Lane k serves the 64-element group k/8: qs word k holds bytes 4(k%8).. of that group; low nibbles are elements
    64(k/8) + 4(k%8).., high nibbles the same + 32; sub-block scales 2(k/8) and 2(k/8)+1."""
    d, dmin = _half_lo(w[0]), _half_hi(w[0])
    sc = w[1:4]
    qh_base, qs_base = (4, 12) if five else (None, 4)
    j = k // 8
    out = []
    vals = []
    for half in (0, 1):
        i_s = 2 * j + half
        wi = i_s // 4
        s, m = _scale_min_6bit(i_s, sc[max(wi, 1) - 1], sc[wi], sc[wi + 1] if wi + 1 < 3 else 0)
        d1 = f32(d * f32(s))
        m1 = f32(dmin * f32(m))
        qs = int(w[qs_base + k])
        q = np.array([(qs >> (8 * b + 4 * half)) & 0xF for b in range(4)], dtype=np.uint32)
        if five:
            qh = int(w[qh_base + (k % 8)])
            u = (1 << (2 * j)) if half == 0 else (2 << (2 * j))
            q = q + np.array([16 if ((qh >> (8 * b)) & u) else 0 for b in range(4)], dtype=np.uint32)
        vals = (q.astype(f32) * d1).astype(f32) - m1
        out.append((64 * j + 32 * half + 4 * (k % 8), vals.astype(f32)))
    return out


def q80x2_lane(w: np.ndarray, k: int):
    """gemv_quant_q8_0x2.slang:27-77, one BlockQ8_0x2 (two GGUF blocks, 17 words) as seen by the 16 lanes that
    share it (k = 0..15): lanes 0-7 take the first block (scale = low half of word 0, int8 data from byte 2 on,
    i.e. words read across a 16-bit shift), lanes 8-15 the second (scale = high half of word 8, data from word 9)."""
    lid = k % 8
    if (k // 8) % 2 == 0:
        scale = _half_lo(w[0])
        data = _i8x4((int(w[lid]) >> 16) | ((int(w[lid + 1]) << 16) & 0xFFFFFFFF))
        first = 4 * lid
    else:
        scale = _half_hi(w[8])
        data = _i8x4(w[lid + 9])
        first = 32 + 4 * lid
    return [(first, (data.astype(f32) * scale).astype(f32))]


def q6kx2_lane(w: np.ndarray, k: int):
    """gemv_quant_q6_kx2.slang:83-172, one BlockQ6Kx2 (two 210-byte blocks, 105 words).  Lanes 0-15 take the first
    block, 16-31 the second, whose fields start on a 16-bit boundary (every word is read across a shift).  Inside a
    block, lane l = k%8 of half i = (k/8)%2 takes ql bytes 4l.. and +32 of that half and qh bytes 4l..: four groups of
    four values at elements 128i + {0,32,64,96} + 4l, scaled by scales[8i + l/4 + {0,2,4,6}] * d."""
    second = k // 16 == 1
    i, l = (k // 8) % 2, k % 8

    def word(idx):  # word idx of this block's own byte stream
        if not second:
            return int(w[idx])
        a = 53 + idx  # (210 bytes = 52.5 words: the second block starts in the high half of word 52)
        return ((int(w[a - 1]) >> 16) | ((int(w[a]) << 16) & 0xFFFFFFFF)) & 0xFFFFFFFF

    d = _half_hi(w[104]) if second else _half_lo(w[52])
    sc0 = (_i8x4(word(48 + 2 * i)).astype(f32) * d).astype(f32)
    sc1 = (_i8x4(word(48 + 2 * i + 1)).astype(f32) * d).astype(f32)
    qh = _u8x4(word(32 + 8 * i + l))
    ql0 = _u8x4(word(16 * i + l))
    ql32 = _u8x4(word(16 * i + l + 8))
    sub = l // 4
    q1 = ((ql0 & 0xF) | ((qh & 3) << 4)).astype(np.int32) - 32
    q2 = ((ql32 & 0xF) | (((qh >> 2) & 3) << 4)).astype(np.int32) - 32
    q3 = ((ql0 >> 4) | (((qh >> 4) & 3) << 4)).astype(np.int32) - 32
    q4 = ((ql32 >> 4) | (((qh >> 6) & 3) << 4)).astype(np.int32) - 32
    base = (256 if second else 0) + 128 * i + 4 * l
    return [(base, (sc0[sub] * q1.astype(f32)).astype(f32)), (base + 32, (sc0[sub + 2] * q2.astype(f32)).astype(f32)),
            (base + 64, (sc1[sub] * q3.astype(f32)).astype(f32)), (base + 96, (sc1[sub + 2] * q4.astype(f32)).astype(f32))]


_FMT = {8: (34, 32, 2), 12: (144, 256, 1), 13: (176, 256, 1), 14: (210, 256, 2)}  # block bytes, elements, blocks per shader unit


def dequantize_rows(fmt: int, blocks: np.ndarray, M: int, K: int) -> np.ndarray:
    """Dense f32 [M, K] assembled through the shaders' lane -> element maps.  K must hold a whole number of shader
    units (Q8_0 and Q6_K shaders work on pairs of blocks)."""
    bb, be, per = _FMT[fmt]
    unit_b, unit_e = bb * per, be * per
    assert K % unit_e == 0
    raw = np.ascontiguousarray(blocks).view(np.uint8).reshape(M, K // unit_e, unit_b)
    out = np.zeros((M, K), dtype=f32)
    seen = np.zeros((M, K), dtype=bool)
    for r in range(M):
        for u in range(K // unit_e):
            pad = (-unit_b) % 4
            w = _words(np.concatenate([raw[r, u], np.zeros(pad, np.uint8)]))
            lanes = range(16) if fmt == 8 else range(32)
            for k in lanes:
                if fmt == 12:
                    parts = q4k_lane(w, k)
                elif fmt == 13:
                    parts = q4k_lane(w, k, five=True)
                elif fmt == 14:
                    parts = q6kx2_lane(w, k)
                else:
                    parts = q80x2_lane(w, k)
                for first, vals in parts:
                    out[r, u * unit_e + first: u * unit_e + first + 4] = vals
                    seen[r, u * unit_e + first: u * unit_e + first + 4] = True
    assert seen.all(), "the lane map does not cover every element"
    return out


def _tree(partials: np.ndarray) -> np.ndarray:
    """reduce_sum(16), (8), (4), (2), (1) over the 32 lanes' partial sums (last axis = lane)."""
    p = partials.astype(f32).copy()
    stride = p.shape[-1] // 2
    while stride >= 1:
        p[..., :stride] = (p[..., :stride] + p[..., stride:2 * stride]).astype(f32)
        stride //= 2
    return p[..., 0]


def gemv(fmt: int, blocks: np.ndarray, v: np.ndarray, M: int, K: int) -> np.ndarray:
    """out = W v in the shaders' summation order: every lane accumulates its own elements block after block (a 4-term
    dot per group of four elements, added to the lane's running sum), then the 32 lane sums meet in a binary tree."""
    W = dequantize_rows(fmt, blocks, M, K)
    bb, be, per = _FMT[fmt]
    unit_e = be * per
    # lane of every element inside a shader unit
    lane_of = np.zeros(unit_e, dtype=np.int64)
    order = []  # (lane, first) in the order a lane visits its groups
    dummy = np.zeros(((bb * per + 3) // 4) * 4, np.uint8)
    if fmt in (12, 13):
        dummy[0:4] = 0
    wd = _words(dummy)
    for k in (range(16) if fmt == 8 else range(32)):
        parts = q4k_lane(wd, k) if fmt == 12 else q4k_lane(wd, k, True) if fmt == 13 else q6kx2_lane(wd, k) if fmt == 14 else q80x2_lane(wd, k)
        for first, _ in parts:
            lanes32 = k if fmt != 8 else k  # Q8_0: lanes 16-31 serve the next pair of the same loop step
            order.append((lanes32, first))
    v = np.asarray(v, dtype=f32)
    acc = np.zeros((M, 32), dtype=f32)
    n_units = K // unit_e
    step_units = 2 if fmt == 8 else 1  # the Q8_0 loop takes two block pairs per step (lanes 0-15 / 16-31)
    for u0 in range(0, n_units, step_units):
        for su in range(step_units):
            u = u0 + su
            if u >= n_units:
                continue
            for lane, first in order:
                ln = lane + (16 * su if fmt == 8 else 0)
                seg = slice(u * unit_e + first, u * unit_e + first + 4)
                prod = (W[:, seg] * v[seg]).astype(f32)
                dot = ((prod[:, 0] + prod[:, 1]).astype(f32) + prod[:, 2]).astype(f32)
                dot = (dot + prod[:, 3]).astype(f32)
                acc[:, ln] = (acc[:, ln] + dot).astype(f32)
    return _tree(acc)


# ---------------------------------------------------------------------------------------------------------
# small operators
# ---------------------------------------------------------------------------------------------------------
def rms_norm(v, w, eps):
    """rms_norm.slang:23-67: 128 lanes add v[i]^2 for i = lane, lane+128, ...; binary tree; out = (v * rms) * w with
    rms = 1 / sqrt(sum / n + eps)."""
    v, w = np.asarray(v, f32), np.asarray(w, f32)
    n = v.size
    part = np.zeros(128, dtype=f32)
    for lane in range(128):
        for i in range(lane, n, 128):
            part[lane] = f32(part[lane] + f32(v[i] * v[i]))
    total = _tree(part[None, :])[0]
    rms = f32(f32(1.0) / np.sqrt(f32(f32(total / f32(n)) + f32(eps))))
    return ((v * rms).astype(f32) * w).astype(f32)


def rope(q, k, head_size, kv_dim, pos, base=10000.0, neox=False):
    """rope.slang:29-54 (adjacent pairs) and :58-86 (NeoX: pairs head_size/2 apart).  Invocation i rotates one pair of
    q (and of k while 2i < kv_dim) by pos * base^(-((2i) mod head_size)/head_size)."""
    q, k = np.asarray(q, f32).copy(), np.asarray(k, f32).copy()
    for i in range(q.size // 2):
        hd = f32((2 * i) % head_size)
        theta = np.power(f32(base), f32(-hd / f32(head_size)), dtype=f32)
        ang = f32(f32(pos) * theta)
        c, s = f32(np.cos(ang, dtype=f32)), f32(np.sin(ang, dtype=f32))
        if neox:
            a = i + ((2 * i) // head_size) * head_size // 2
            b = a + head_size // 2
        else:
            a, b = 2 * i, 2 * i + 1
        for vec, active in ((q, True), (k, 2 * i < kv_dim)):
            if not active:
                continue
            x, y = vec[a], vec[b]
            vec[a] = f32(f32(c * x) - f32(s * y))
            vec[b] = f32(f32(s * x) + f32(c * y))
    return q, k


def softmax(col):
    """softmax.slang:26-96 on one column: 64 lanes take the maximum / the sum of exp(x - max) over i = lane, lane+64, ...;
    binary trees; every element divided by the sum."""
    x = np.asarray(col, f32)
    n = x.size
    mx = np.full(64, f32(-1.0e38), dtype=f32)
    for lane in range(64):
        for i in range(lane, n, 64):
            mx[lane] = max(mx[lane], x[i])
    stride = 32
    while stride >= 1:
        mx[:stride] = np.maximum(mx[:stride], mx[stride:2 * stride])
        stride //= 2
    e = np.exp((x - mx[0]).astype(f32), dtype=f32)
    part = np.zeros(64, dtype=f32)
    for lane in range(64):
        for i in range(lane, n, 64):
            part[lane] = f32(part[lane] + e[i])
    den = _tree(part[None, :])[0]
    return (e / den).astype(f32)


def attention(q, key_cache, value_cache, kv_mul, n_heads, head_size, pos):
    """ops/batched_multiquery_attention.rs:43-98 with batched_multiquery_attention.slang:18-32: scores = K^T q for
    positions 0..=pos (padded rows up to a multiple of four are zeroed by the mask kernel and left out of the softmax),
    divided by sqrt(head_size) AFTER the product; column softmax; xb = V att.  Caches are [positions, kv_dim]."""
    q = np.asarray(q, f32)
    out = np.zeros(n_heads * head_size, dtype=f32)
    for h in range(n_heads):
        kvh = h // kv_mul
        ks = np.asarray(key_cache, f32)[: pos + 1, kvh * head_size:(kvh + 1) * head_size]
        vs = np.asarray(value_cache, f32)[: pos + 1, kvh * head_size:(kvh + 1) * head_size]
        qh = q[h * head_size:(h + 1) * head_size]
        scores = np.zeros(pos + 1, dtype=f32)
        for t in range(pos + 1):
            acc = f32(0)
            for j in range(head_size):
                acc = f32(acc + f32(ks[t, j] * qh[j]))
            scores[t] = f32(acc / np.sqrt(f32(head_size)))
        att = softmax(scores)
        acc = np.zeros(head_size, dtype=f32)
        for t in range(pos + 1):
            acc = (acc + (vs[t] * att[t]).astype(f32)).astype(f32)
        out[h * head_size:(h + 1) * head_size] = acc
    return out
