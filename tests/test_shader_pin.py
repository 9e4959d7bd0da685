"""Pins the oracle a second way: against a numpy restatement of the reference's Slang shaders
(tests/shader_restatement.py), an independent description of the same operators inside the reference.  The
reference stores no golden vectors for GEMV, norms, RoPE, softmax or attention; two of its own descriptions agreeing
(CPU operator path = the oracle, GPU shaders = the restatement) is the strongest pin available without running it.
Dequantised values must agree bit for bit; sums within the rounding of their different summation orders."""
import numpy as np
import pytest

import shader_restatement as S
from oracle import oracle as O
from slai_b200 import synth
from helpers import bits, rel_l2

FMTS = [synth.FMT_Q8_0, synth.FMT_Q4_K, synth.FMT_Q5_K, synth.FMT_Q6_K]


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("kind", ["quantized", "random_bits"])
def test_shader_lane_maps_dequantise_like_the_cpu_blocks(fmt, kind):
    M, K = 4, 1024 if fmt != synth.FMT_Q8_0 else 256
    rng = np.random.default_rng(fmt)
    blocks = synth.quantize(fmt, synth.normal_matrix(fmt, M, K)) if kind == "quantized" else synth.random_blocks(fmt, M, K, rng)
    got = S.dequantize_rows(fmt, blocks, M, K)
    want = O.dequantize(fmt, blocks).reshape(M, K)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("fmt", FMTS)
def test_shader_gemv_order_agrees_with_the_oracle(fmt):
    M, K = 8, 2048 if fmt != synth.FMT_Q8_0 else 512
    blocks = synth.quantize(fmt, synth.normal_matrix(7 + fmt, M, K))
    v = np.random.default_rng(fmt).standard_normal(K).astype(np.float32)
    got = S.gemv(fmt, blocks, v, M, K)
    W = O.dequantize(fmt, blocks).reshape(M, K)
    exact = W.astype(np.float64) @ v.astype(np.float64)
    assert rel_l2(got, exact) < 2e-6                                  # f32, lane-wise then tree
    assert rel_l2(O.gemv_f32(W, v), exact) < 2e-6                     # f32, sequential (the CPU twin)
    assert rel_l2(O.gemv_quant(fmt, blocks, v, M, K), exact) < 2e-6   # the oracle's fused form
    assert rel_l2(got, O.gemv_f32(W, v)) < 3e-6


@pytest.mark.parametrize("n,eps", [(288, 1e-5), (1757, 1e-5), (4096, 1e-6)])
def test_shader_rms_norm(n, eps):
    rng = np.random.default_rng(n)
    v, w = rng.standard_normal(n).astype(np.float32), rng.uniform(0.5, 1.5, n).astype(np.float32)
    assert np.allclose(S.rms_norm(v, w, eps), O.rms_norm(v, w, eps), rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("pos", [0, 10, 4095])
def test_shader_rope(neox, pos):
    rng = np.random.default_rng(pos)
    hs, dim, kvd = 64, 256, 128
    q, k = rng.standard_normal(dim).astype(np.float32), rng.standard_normal(kvd).astype(np.float32)
    gq, gk = S.rope(q, k, hs, kvd, pos, neox=neox)
    wq, wk = O.rope(q, k, hs, kvd, pos, neox=neox)
    # The angle pos * theta is as large as pos radians: a one-ulp difference between the two pow() implementations
    # (numpy here, libm in the oracle) moves it by up to pos * 1.2e-7 radians.  That is the conditioning of the
    # formula, not a difference of method; the bound scales with the position (1e-5 at position 0).
    atol = 1e-5 + 4e-7 * pos
    assert np.allclose(gq, wq, atol=atol) and np.allclose(gk, wk, atol=atol)


def test_shader_softmax_and_attention():
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(1000) * 4).astype(np.float32)
    assert np.allclose(S.softmax(x), O.softmax(x), rtol=5e-6, atol=1e-10)
    seq, nh, kvm, hs, pos = 64, 6, 3, 48, 37   # the shapes of the reference's own (disabled) attention test
    kvd = nh // kvm * hs
    q = rng.standard_normal(nh * hs).astype(np.float32)
    kc, vc = rng.standard_normal((seq, kvd)).astype(np.float32), rng.standard_normal((seq, kvd)).astype(np.float32)
    got = S.attention(q, kc, vc, kvm, nh, hs, pos)
    want, _ = O.attention(q, kc, vc, seq_len=seq, kv_dim=kvd, kv_mul=kvm, n_heads=nh, head_size=hs, pos=pos)
    assert rel_l2(got, want) < 2e-6
