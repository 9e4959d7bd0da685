"""CPU tests of the oracle (no GPU): golden block recipes, an independent dequantiser, and the operator twins
against float64 numpy formulas."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import synth

GOLD = os.path.join(os.path.dirname(__file__), "golden")
FMTS = [synth.FMT_Q8_0, synth.FMT_Q4_K, synth.FMT_Q5_K, synth.FMT_Q6_K]


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("fmt", FMTS)
def test_block_recipes_bit_exact(fmt):
    g = np.load(os.path.join(GOLD, "block_recipes.npz"))
    name = synth.FMT_NAMES[fmt]
    got = O.dequantize(fmt, g[f"{name}_blocks"])
    assert np.array_equal(bits(got), bits(g[f"{name}_values"]))


def test_recipe_spot_values():
    """Hand-computed entries of the reference's recipe blocks (ops/quantization.rs:78-83, 204-220)."""
    g = np.load(os.path.join(GOLD, "block_recipes.npz"))
    s = np.float32(np.float16(1.234))
    v = g["q8_0_values"].reshape(8, 32)
    assert v[0, 0] == np.float32(-128) * s and v[3, 5] == np.float32(3 * 16 - 128 + 5) * s
    # Q6_K block 0: d = f16 bits 123 (subnormal 123 * 2^-24), scale[0] = -127, ql[0] = 0, qh[0] = 0 -> q = -32
    d = np.float32(123 * 2.0 ** -24)
    assert g["q6_k_values"][0] == (d * np.float32(-127)) * np.float32(-32)
    # Q4_K block 1: scales[k] = 16 + k; sub-block 0: sc = 16 & 63, m = scales[4] & 63 = 20; qs[0] = 16 -> low nibble 0
    d4, m4 = np.float32(np.float16(1.234)), np.float32(np.float16(5.678))
    assert g["q4_k_values"][256] == (d4 * np.float32(16)) * np.float32(0) - m4 * np.float32(20)


@pytest.mark.parametrize("fmt", FMTS)
def test_dequantize_vs_gguf_package(fmt):
    gguf = pytest.importorskip("gguf")
    from gguf import quants, GGMLQuantizationType as T
    t = {synth.FMT_Q8_0: T.Q8_0, synth.FMT_Q4_K: T.Q4_K, synth.FMT_Q5_K: T.Q5_K, synth.FMT_Q6_K: T.Q6_K}[fmt]
    rng = np.random.default_rng(fmt)
    for blocks in (synth.quantize(fmt, synth.normal_matrix(fmt, 6, 1024)), synth.random_blocks(fmt, 5, 768 if fmt != synth.FMT_Q8_0 else 96, rng)):
        ours = O.dequantize(fmt, blocks)
        ref = quants.dequantize(blocks, t).reshape(-1).astype(np.float32)
        assert np.array_equal(bits(ours), bits(ref))


def test_f16_codec_exhaustive():
    allh = np.arange(65536, dtype=np.uint16)
    dec = np.array([O.decode_f16(int(h)) for h in allh], dtype=np.float32)
    ref = allh.view(np.float16).astype(np.float32)
    same = (dec == ref) | (np.isnan(dec) & np.isnan(ref))
    assert same.all()
    x = np.concatenate([np.random.default_rng(0).standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-6, 1e-4, 1, 300, 7e4)])
    enc = np.array([O.encode_f16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(enc, x.astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("fmt", FMTS)
def test_quantizers_make_valid_blocks(fmt):
    x = synth.normal_matrix(7, 4, 512)
    dq = O.dequantize(fmt, synth.quantize(fmt, x)).reshape(4, 512)
    rel = np.linalg.norm(dq - x) / np.linalg.norm(x)
    assert np.isfinite(dq).all() and rel < {synth.FMT_Q8_0: 0.01, synth.FMT_Q4_K: 0.12, synth.FMT_Q5_K: 0.06, synth.FMT_Q6_K: 0.04}[fmt]
    z = O.dequantize(fmt, synth.quantize(fmt, np.zeros((1, 256), np.float32)))
    assert np.all(z == 0)


def test_gemv_matches_f64_and_threads():
    rng = np.random.default_rng(3)
    w = rng.standard_normal((37, 1757), dtype=np.float32)
    x = rng.standard_normal(1757, dtype=np.float32)
    a, b, c = O.gemv_f32(w, x), O.gemv_f32(w, x, nthreads=4), O.gemv_f64acc(w, x)
    assert np.array_equal(a, b)
    assert np.linalg.norm(a - c) / np.linalg.norm(c) < 1e-5
    blocks = synth.quantize(synth.FMT_Q4_K, rng.standard_normal((9, 512), dtype=np.float32))
    v = rng.standard_normal(512, dtype=np.float32)
    ref = O.dequantize(synth.FMT_Q4_K, blocks).reshape(9, 512).astype(np.float64) @ v.astype(np.float64)
    got = O.gemv_quant(synth.FMT_Q4_K, blocks, v, 9, 512, nthreads=2)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 1e-5


def test_small_ops_vs_numpy():
    rng = np.random.default_rng(5)
    n = 1757  # the size the reference's operator tests use
    a, w = rng.random(n, dtype=np.float32), rng.random(n, dtype=np.float32)
    a64 = a.astype(np.float64)
    np.testing.assert_allclose(O.rms_norm(a, w), a64 / np.sqrt((a64 ** 2).mean() + 1e-5) * w, rtol=2e-6)
    np.testing.assert_allclose(O.layernorm(a), (a64 - a64.mean()) / np.sqrt(a64.var() + 1e-5), rtol=1e-4, atol=1e-6)
    e = np.exp(a64 - a64.max())
    np.testing.assert_allclose(O.softmax(a), e / e.sum(), rtol=1e-5)
    h2 = rng.standard_normal(n).astype(np.float32)
    x = (a - 0.5) * 8
    np.testing.assert_allclose(O.silu_gate(x, h2), h2 * (x.astype(np.float64) / (1 + np.exp(-x.astype(np.float64)))), rtol=1e-5, atol=1e-7)
    g = 0.5 * x.astype(np.float64) * (1 + np.tanh(0.7978846 * x * (1 + 0.044715 * x.astype(np.float64) ** 2)))
    np.testing.assert_allclose(O.unary("gelu", x), g, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(O.unary("scale", x, (2.5,)), x * np.float32(2.5))
    np.testing.assert_allclose(O.unary("clamp", x, (-1.0, 2.0)), np.clip(x, -1, 2))
    assert O.argmax(np.array([1, 5, 5, 2], np.float32)) == 1  # first maximal index


def test_rope_variants():
    rng = np.random.default_rng(9)
    hs, nq, nk, pos = 128, 13, 9, 10  # the shapes of the reference's RoPE test (ops/rope.rs:144-228)
    q, k = rng.random(nq * hs, dtype=np.float32), rng.random(nk * hs, dtype=np.float32)
    kk = np.concatenate([k, np.zeros((nq - nk) * hs, np.float32)])
    q2, k2 = O.rope(q, kk, hs, nk * hs, pos)
    i = np.arange(0, nq * hs, 2)
    th = 10000.0 ** (-(i % hs) / hs) * pos
    np.testing.assert_allclose(q2[i], np.cos(th) * q[i] - np.sin(th) * q[i + 1], atol=2e-5)
    np.testing.assert_allclose(q2[i + 1], np.sin(th) * q[i] + np.cos(th) * q[i + 1], atol=2e-5)
    assert np.array_equal(k2[nk * hs:], kk[nk * hs:])  # untouched beyond kv_dim
    np.testing.assert_allclose(k2[:nk * hs:2], (np.cos(th) * kk[i] - np.sin(th) * kk[i + 1])[: nk * hs // 2], atol=2e-5)
    # NeoX pairs are head_size/2 apart; norms of pairs are preserved
    q3, _ = O.rope(q, kk, hs, nk * hs, pos, neox=True)
    qa, qb = q.reshape(nq, 2, hs // 2), q3.reshape(nq, 2, hs // 2)
    np.testing.assert_allclose(qa[:, 0] ** 2 + qa[:, 1] ** 2, qb[:, 0] ** 2 + qb[:, 1] ** 2, rtol=1e-4)
    np.testing.assert_allclose(qb[:, 0, 0], np.cos(0.0 * pos + pos * 1.0) * qa[:, 0, 0] - np.sin(pos * 1.0) * qa[:, 1, 0], atol=2e-5)


def test_attention_vs_numpy():
    rng = np.random.default_rng(11)
    # the shapes of the reference's (disabled) attention test: seq 1024, kv_dim 768, 12 heads of 64
    seq, hs, nh, kv_mul = 1024, 64, 12, 1
    kv_dim = nh // kv_mul * hs
    for pos, kvm in ((0, 1), (7, 1), (100, 3)):
        nkv = nh // kvm
        kvd = nkv * hs
        q = rng.standard_normal(nh * hs).astype(np.float32)
        kc = rng.standard_normal((seq, kvd)).astype(np.float32)
        vc = rng.standard_normal((seq, kvd)).astype(np.float32)
        xb, _ = O.attention(q, kc, vc, seq_len=seq, kv_dim=kvd, kv_mul=kvm, n_heads=nh, head_size=hs, pos=pos)
        for h in range(nh):
            kh = kc[: pos + 1, (h // kvm) * hs:(h // kvm + 1) * hs].astype(np.float64)
            vh = vc[: pos + 1, (h // kvm) * hs:(h // kvm + 1) * hs].astype(np.float64)
            s = kh @ q[h * hs:(h + 1) * hs] / np.sqrt(hs)
            p = np.exp(s - s.max())
            p /= p.sum()
            np.testing.assert_allclose(xb[h * hs:(h + 1) * hs], p @ vh, rtol=2e-4, atol=2e-5)


def test_tiny_llama_fixture_reproduces():
    """The tiny-Llama benchmark configuration through the oracle reproduces the committed greedy ids (first 24 steps checked here;
    tests/golden/make_golden.py wrote all 128)."""
    from slai_b200.models import TINY_LLAMA as cfg, synthetic_llama_host
    g = np.load(os.path.join(GOLD, "tiny_llama_greedy.npz"))
    w = synthetic_llama_host(cfg, synth.FMT_Q8_0, seed=int(g["seed"][0]))
    model = O.Llama(dim=cfg.dim, hidden=cfg.hidden_dim, n_layers=cfg.n_layers, n_q=cfg.n_q_heads, n_kv=cfg.n_kv_heads,
                    vocab=cfg.vocab_size, seq_len=cfg.seq_len, eps=cfg.rms_norm_eps, nthreads=4)
    shapes = cfg.matrix_shapes()
    for (name, l), val in w.items():
        if name in shapes:
            model.set_weight(name, l, O.dequantize(synth.FMT_Q8_0, val).reshape(shapes[name]))
        elif name == "output":
            model.set_weight(name, l, O.dequantize(synth.FMT_Q8_0, val).reshape(cfg.vocab_size, cfg.dim))
        else:
            model.set_weight(name, l, val)
    prompt = g["prompt"]
    tok, got = int(prompt[0]), []
    for pos in range(16 + 24 - 1):
        logits = model.forward(tok, pos)
        tok = int(prompt[pos + 1]) if pos + 1 < 16 else O.argmax(logits)
        if pos + 1 >= 16:
            got.append(tok)
    assert got == list(g["tokens"][:24])
