"""Prompt processing as tensor-core GEMMs (slai_llama_prefill with 16 tokens or more) against the sequential path (the
same prompt fed through the decode step token by token, which is what the reference does) and against the oracle:
logits of the last prompt token and the KV cache within 1e-3 relative L2, same greedy continuation."""
import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import synth, _lib
from slai_b200.models import Llama2Config, llama_from_host, synthetic_llama_host
from helpers import oracle_llama, rel_l2

pytestmark = pytest.mark.gpu


def _models(backend, monkeypatch, cfg, fmt, out_fmt, seed):
    w = synthetic_llama_host(cfg, fmt, out_fmt, seed=seed, std=0.05, embd_std=1.0)
    batched = llama_from_host(backend, cfg, w, fmt, out_fmt)
    seq = llama_from_host(backend, cfg, w, fmt, out_fmt)
    return w, batched, seq


@pytest.mark.parametrize("T", [16, 100, 512])
@pytest.mark.parametrize("fmt,out_fmt,kv_dtype", [(synth.FMT_Q4_K, synth.FMT_Q6_K, _lib.KV_F16), (synth.FMT_Q8_0, synth.FMT_Q8_0, _lib.KV_F32)])
def test_batched_prefill_matches_sequential(backend, monkeypatch, T, fmt, out_fmt, kv_dtype):
    cfg = Llama2Config(dim=512, hidden_dim=1280, n_layers=3, n_q_heads=8, n_kv_heads=2, vocab_size=2000, seq_len=640, kv_dtype=kv_dtype)
    w, batched, seq = _models(backend, monkeypatch, cfg, fmt, out_fmt, seed=T)
    prompt = np.random.default_rng(T).integers(0, cfg.vocab_size, size=T).astype(np.int32)
    lg_b = batched.prefill(prompt, 0, want_logits=True)
    monkeypatch.setenv("SLAI_PREFILL_SEQUENTIAL", "1")
    lg_s = seq.prefill(prompt, 0, want_logits=True)
    monkeypatch.delenv("SLAI_PREFILL_SEQUENTIAL")
    assert np.isfinite(lg_b).all()
    assert rel_l2(lg_b, lg_s) < 1e-3, rel_l2(lg_b, lg_s)
    for layer in (0, cfg.n_layers - 1):
        kb, vb = batched.read_kv(layer, T)
        ks, vs = seq.read_kv(layer, T)
        assert rel_l2(kb, ks) < 1e-3 and rel_l2(vb, vs) < 1e-3, (layer, rel_l2(kb, ks), rel_l2(vb, vs))
    # same greedy continuation (both models continue through the decode step, on their own caches)
    first = int(np.argmax(lg_s))
    top2 = np.partition(lg_s, -2)[-2:]
    if top2[1] - top2[0] > 1e-3 * np.abs(lg_s).max():
        assert int(np.argmax(lg_b)) == first
    gb = batched.generate(first, T, 24)
    gs = seq.generate(first, T, 24)
    agree = 0
    for a, b in zip(gb, gs):
        if a != b:
            break
        agree += 1
    assert agree >= 12, (list(gb), list(gs))   # ids may part only where the top two logits are within rounding of each other


def test_batched_prefill_matches_oracle(backend):
    """Against the CPU oracle directly (not only against the other CUDA path), at a non-zero start position after a
    short sequential prompt: logits of the last token within 1e-3."""
    cfg = Llama2Config(dim=512, hidden_dim=1280, n_layers=2, n_q_heads=8, n_kv_heads=4, vocab_size=1500, seq_len=128, kv_dtype=_lib.KV_F32)
    w = synthetic_llama_host(cfg, synth.FMT_Q4_K, synth.FMT_Q4_K, seed=9, std=0.05, embd_std=1.0)
    m = llama_from_host(backend, cfg, w, synth.FMT_Q4_K, synth.FMT_Q4_K)
    ref = oracle_llama(cfg, w, synth.FMT_Q4_K, synth.FMT_Q4_K)
    rng = np.random.default_rng(1)
    head, tail = rng.integers(0, cfg.vocab_size, size=5).astype(np.int32), rng.integers(0, cfg.vocab_size, size=40).astype(np.int32)
    m.prefill(head, 0)                                   # 5 tokens: the decode step
    got = m.prefill(tail, len(head), want_logits=True)   # 40 tokens from position 5: the GEMM path, attending to the first 5
    want = None
    for pos, tok in enumerate(list(head) + list(tail)):
        want = ref.forward(int(tok), pos)
    assert rel_l2(got, want) < 1e-3, rel_l2(got, want)


def test_prefill_falls_back_for_short_prompts_and_odd_widths(backend):
    """Fewer than 16 tokens, or a column count that is not a multiple of 64, go through the decode step: bit-identical
    to feeding the tokens one by one."""
    cfg = Llama2Config(dim=288, hidden_dim=768, n_layers=2, n_q_heads=6, n_kv_heads=6, vocab_size=500, seq_len=64, kv_dtype=_lib.KV_F32)
    w = synthetic_llama_host(cfg, synth.FMT_Q8_0, seed=2, std=0.05, embd_std=1.0)
    a = llama_from_host(backend, cfg, w, synth.FMT_Q8_0)
    b = llama_from_host(backend, cfg, w, synth.FMT_Q8_0)
    prompt = np.random.default_rng(0).integers(0, cfg.vocab_size, size=20).astype(np.int32)
    la = a.prefill(prompt, 0, want_logits=True)   # dim 288 is not a multiple of 64
    for pos, t in enumerate(prompt):
        lb, _ = b.forward_logits(pos, int(t))
    assert np.array_equal(la, lb)


@pytest.mark.parametrize("kv_dtype,n_embd,n_head", [(_lib.KV_F16, 256, 4), (_lib.KV_F32, 192, 3)])
def test_gpt2_prompt_pass_matches_the_sequential_pass_and_the_oracle(backend, monkeypatch, kv_dtype, n_embd, n_head):
    """GPT-2's prompt pass as GEMMs (LayerNorm + bias + GELU variants of the Llama pass): last logits against the oracle fed
    token by token and against the library's own sequential pass, same greedy continuation, continuing from a later
    position too."""
    from slai_b200.models import Gpt2Params, gpt2_from_host, synthetic_gpt2_host
    from helpers import oracle_gpt2
    p = Gpt2Params(n_vocab=700, n_seq=96, n_embd=n_embd, n_head=n_head, n_layer=2, ff_len=4 * n_embd, kv_dtype=kv_dtype)
    w = synthetic_gpt2_host(p, seed=6, std=0.08, bias_std=0.05)
    rng = np.random.default_rng(8)
    prompt = rng.integers(0, p.n_vocab, size=40).astype(np.int32)
    batched = gpt2_from_host(backend, p, w)
    lg_b = batched.prefill(prompt, 0, want_logits=True)
    ref = oracle_gpt2(p, w, kv_f16=(kv_dtype == _lib.KV_F16))
    for pos, t in enumerate(prompt):
        want = ref.forward(int(t), pos)
    assert rel_l2(lg_b, want) < 1e-3
    monkeypatch.setenv("SLAI_PREFILL_SEQUENTIAL", "1")
    seq = gpt2_from_host(backend, p, w)
    lg_s = seq.prefill(prompt, 0, want_logits=True)
    monkeypatch.delenv("SLAI_PREFILL_SEQUENTIAL")
    assert rel_l2(lg_b, lg_s) < 1e-3
    tok = int(np.argmax(lg_s))
    assert list(batched.generate(tok, 40, 20)) == list(seq.generate(tok, 40, 20))
    # a second block of the prompt from position 60 on (attends to everything before it)
    more = rng.integers(0, p.n_vocab, size=20).astype(np.int32)
    la = batched.prefill(more, 60, want_logits=True)
    monkeypatch.setenv("SLAI_PREFILL_SEQUENTIAL", "1")
    lb = seq.prefill(more, 60, want_logits=True)
    monkeypatch.delenv("SLAI_PREFILL_SEQUENTIAL")
    assert rel_l2(la, lb) < 1e-3
