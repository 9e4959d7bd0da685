"""The legacy block formats (Q4_0, Q4_1, Q5_0, Q5_1, Q8_K: crates/slai/src/quantization.rs:47-199) and the NeoX RoPE
variant (rope.slang:58-86) through the C ABI: dequantised values bit-exact against the oracle on the reference's
recipes and on random bit patterns, GEMV and whole models within 1e-3."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import synth, _lib
from slai_b200.models import Llama2Config, llama_from_host, synthetic_llama_host
from slai_b200.ops import GpuQuantMatrix
from helpers import bits, oracle_llama, rel_l2

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
LEGACY = list(synth.LEGACY_FORMATS)


@pytest.mark.parametrize("fmt", LEGACY)
def test_legacy_recipes_dequantise_bit_exact(backend, fmt):
    g = np.load(os.path.join(GOLD, "block_recipes.npz"))
    name = synth.FMT_NAMES[fmt]
    blocks = g[f"{name}_blocks"]
    nb, be = blocks.shape[0], synth.BLOCK_ELEMS[fmt]
    for rows in (1, 4, 16):
        m = GpuQuantMatrix(backend, fmt, rows, nb // rows * be, blocks)
        assert np.array_equal(bits(m.dequantize().reshape(-1)), bits(g[f"{name}_values"]))
    f, r, c = C.c_int(), C.c_int64(), C.c_int64()
    backend.check(backend.lib.slai_qmatrix_shape(m.h, C.byref(f), C.byref(r), C.byref(c)))
    assert f.value == fmt   # the handle reports the format that was uploaded, whatever the device representation


@pytest.mark.parametrize("fmt", LEGACY)
def test_legacy_random_blocks_and_gemv(backend, ctx, fmt):
    M, K = 70, 1024
    rng = np.random.default_rng(fmt)
    for blocks in (synth.random_blocks(fmt, M, K, rng), synth.quantize(fmt, synth.normal_matrix(fmt, M, K))):
        m = GpuQuantMatrix(backend, fmt, M, K, blocks)
        want = O.dequantize(fmt, blocks)
        assert np.array_equal(bits(m.dequantize().reshape(-1)), bits(want))
        assert np.array_equal(bits(m.dequantize_row(M - 1)), bits(want.reshape(M, K)[M - 1]))
        v = rng.standard_normal(K).astype(np.float32)
        out = backend.zeros(M)
        ctx.matmul_quant_assign(out, m, backend.vector(v))
        ref = want.reshape(M, K).astype(np.float64) @ v.astype(np.float64)
        assert rel_l2(out.to_numpy(), ref) < 1e-5


@pytest.mark.parametrize("fmt", [synth.FMT_Q4_0, synth.FMT_Q4_1, synth.FMT_Q8_K])
def test_llama_with_legacy_layers_matches_oracle(backend, fmt):
    """Q4_0 runs through the fused decode kernels (as Q8_0 blocks), Q4_1 / Q8_K through the operator-by-operator layer on
    dense f32 matrices; both against the oracle on the uploaded blocks."""
    cfg = Llama2Config(dim=256, hidden_dim=512, n_layers=2, n_q_heads=4, n_kv_heads=2, vocab_size=400, seq_len=48, kv_dtype=_lib.KV_F32)
    w = synthetic_llama_host(cfg, fmt, synth.FMT_Q8_0, seed=7, std=0.05, embd_std=1.0)
    m = llama_from_host(backend, cfg, w, fmt, synth.FMT_Q8_0)
    ref = oracle_llama(cfg, w, fmt, synth.FMT_Q8_0)
    tok = 5
    for pos in range(12):
        lg, nxt = m.forward_logits(pos, tok)
        rl = ref.forward(tok, pos)
        assert rel_l2(lg, rl) < 1e-3, pos
        tok = O.argmax(rl)
    toks = m.generate(tok, 12, 20)   # the same path inside the replayed graph, position on the device
    want = []
    for i in range(20):
        rl = ref.forward(tok, 12 + i)
        tok = O.argmax(rl)
        want.append(tok)
    agree = sum(1 for a, b in zip(toks, want) if a == b)
    assert agree >= 15, (list(toks), want)


@pytest.mark.parametrize("fmt,kv_dtype,biases", [(synth.FMT_Q4_K, _lib.KV_F16, False), (synth.FMT_Q8_0, _lib.KV_F32, True)])
def test_neox_llama_matches_oracle(backend, fmt, kv_dtype, biases):
    """Qwen2-style model: NeoX rotation (pairs half a head apart) and q / k / v biases, through the fused decode path and
    through the GEMM prompt path."""
    cfg = Llama2Config(dim=512, hidden_dim=1024, n_layers=2, n_q_heads=8, n_kv_heads=2, vocab_size=700, seq_len=96, rope_variant=1,
                       kv_dtype=kv_dtype)
    w = synthetic_llama_host(cfg, fmt, fmt, seed=13, std=0.05, embd_std=1.0)
    if biases:
        rng = np.random.default_rng(2)
        for l in range(cfg.n_layers):
            w[("bq", l)] = (0.1 * rng.standard_normal(cfg.dim)).astype(np.float32)
            w[("bk", l)] = (0.1 * rng.standard_normal(cfg.kv_dim)).astype(np.float32)
            w[("bv", l)] = (0.1 * rng.standard_normal(cfg.kv_dim)).astype(np.float32)
    m = llama_from_host(backend, cfg, w, fmt, fmt)
    ref = oracle_llama(cfg, w, fmt, fmt, kv_f16=(kv_dtype == _lib.KV_F16))
    prompt = np.random.default_rng(3).integers(0, cfg.vocab_size, size=20).astype(np.int32)
    tok = int(prompt[0])
    for pos in range(30):
        lg, nxt = m.forward_logits(pos, tok)
        rl = ref.forward(tok, pos)
        assert rel_l2(lg, rl) < 1e-3, pos
        tok = int(prompt[pos + 1]) if pos + 1 < len(prompt) else O.argmax(rl)
    # the prompt through the tensor-core path on a second model: logits of its last token against the oracle
    m2 = llama_from_host(backend, cfg, w, fmt, fmt)
    ref2 = oracle_llama(cfg, w, fmt, fmt, kv_f16=(kv_dtype == _lib.KV_F16))
    got = m2.prefill(prompt, 0, want_logits=True)
    for pos, t in enumerate(prompt):
        want = ref2.forward(int(t), pos)
    assert rel_l2(got, want) < 1e-3
