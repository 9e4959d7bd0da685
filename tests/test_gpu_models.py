"""GPU parity of the decode path (Llama-2 and GPT-2) against the CPU oracle built from the same block bytes:
logits within 1e-3 relative L2, greedy token ids identical."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import synth, _lib
from slai_b200.models import (GPT2_TINY, TINY_LLAMA, Gpt2Params, Llama2Config, gpt2_from_host, llama_from_host,
                              synthetic_gpt2_host, synthetic_llama_host)
from helpers import oracle_gpt2, oracle_llama, rel_l2

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_tiny_llama_greedy_matches_fixture(backend):
    """The tiny-Llama benchmark configuration: 16-token prompt, 128 greedy tokens, Q8_0; ids equal the committed oracle run."""
    g = np.load(os.path.join(GOLD, "tiny_llama_greedy.npz"))
    cfg = Llama2Config(**{**TINY_LLAMA.__dict__, "kv_dtype": _lib.KV_F32})
    w = synthetic_llama_host(cfg, synth.FMT_Q8_0, seed=int(g["seed"][0]))
    m = llama_from_host(backend, cfg, w, synth.FMT_Q8_0)
    prompt = g["prompt"]
    logits = m.prefill(prompt[:-1], 0)
    toks = m.generate(int(prompt[-1]), len(prompt) - 1, 128)
    assert list(toks[:64]) == list(g["tokens"][:64])
    assert list(toks) == list(g["tokens"])
    # the same through per-token calls with logits read back (the reference's forward_logits loop)
    m2 = llama_from_host(backend, cfg, w, synth.FMT_Q8_0)
    tok, got = int(prompt[0]), []
    for pos in range(16 + 8 - 1):
        lg, nxt = m2.forward_logits(pos, tok)
        assert nxt == int(np.argmax(lg))
        tok = int(prompt[pos + 1]) if pos + 1 < 16 else nxt
        if pos + 1 >= 16:
            got.append(tok)
    assert got == list(g["tokens"][:8])


@pytest.mark.parametrize("which", ["7b", "70b"])
def test_headline_shape_llama_matches_the_oracle_fixture(backend, which):
    """Llama at the headline dimensions (7B: dim 4096 / FFN 11008 / 32 heads x 128 / vocab 32000, 2 layers, 64-token
    prompt; 70B: dim 8192 / FFN 28672 / 64 query + 8 KV heads, 1 layer, 16-token prompt), Q4_K + Q6_K logits, fp16 KV:
    logits of the last prompt token within 1e-3 relative L2 of the committed oracle run and the first 64 greedy ids
    identical (tests/golden/make_shape_golden.py wrote the fixture and chose the seed; the smallest top-1/top-2
    margin of the run is stored with it)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_shape_golden", os.path.join(GOLD, "make_shape_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    g = np.load(os.path.join(GOLD, gen.SHAPES[which]["file"]))
    cfg = gen.config(which)
    w = gen.weights(which, int(g["seed"][0]))
    m = llama_from_host(backend, cfg, w, synth.FMT_Q4_K, synth.FMT_Q6_K)
    del w
    prompt = g["prompt"]
    logits = m.prefill(prompt, 0, want_logits=True)
    assert rel_l2(logits, g["last_prompt_logits"]) < 1e-3
    first = int(np.argmax(logits))
    assert first == int(g["tokens"][0])
    toks = m.generate(first, len(prompt), 63)
    assert float(g["margins"].min()) > 4e-4          # the ids are pinned: top two logits clearly apart at every step
    assert [first] + list(toks) == list(g["tokens"][:64])


@pytest.mark.parametrize("fmt,out_fmt", [(synth.FMT_Q4_K, synth.FMT_Q6_K), (synth.FMT_Q5_K, synth.FMT_Q5_K), (synth.FMT_Q8_0, synth.FMT_Q8_0)])
@pytest.mark.parametrize("kv_dtype", [_lib.KV_F32, _lib.KV_F16])
def test_small_llama_logits_and_tokens(backend, fmt, out_fmt, kv_dtype):
    """A small GQA Llama (K-quant block sizes need dims that are multiples of 256)."""
    cfg = Llama2Config(dim=512, hidden_dim=1280, n_layers=3, n_q_heads=8, n_kv_heads=2, vocab_size=2000, seq_len=96, kv_dtype=kv_dtype)
    w = synthetic_llama_host(cfg, fmt, out_fmt, seed=3, std=0.05, embd_std=1.0)
    m = llama_from_host(backend, cfg, w, fmt, out_fmt)
    ref = oracle_llama(cfg, w, fmt, out_fmt, kv_f16=(kv_dtype == _lib.KV_F16))
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab_size, size=12)
    tok = int(prompt[0])
    n_match = 0
    for pos in range(40):
        lg, nxt = m.forward_logits(pos, tok)
        rl = ref.forward(tok, pos)
        assert rel_l2(lg, rl) < 1e-3, pos
        assert rel_l2(m.read_state("x"), ref.x()) < 1e-3
        if pos + 1 < len(prompt):
            tok = int(prompt[pos + 1])
        else:
            top2 = np.partition(rl, -2)[-2:]
            if top2[1] - top2[0] > 1e-4 * np.abs(rl).max():
                assert nxt == O.argmax(rl), pos
                n_match += 1
            tok = O.argmax(rl)
    assert n_match > 10


def test_llama_prefill_generate_equals_stepwise(backend):
    cfg = Llama2Config(dim=256, hidden_dim=512, n_layers=2, n_q_heads=4, n_kv_heads=4, vocab_size=500, seq_len=64)
    w = synthetic_llama_host(cfg, synth.FMT_Q4_K, seed=5, std=0.05, embd_std=1.0)
    a = llama_from_host(backend, cfg, w, synth.FMT_Q4_K)
    b = llama_from_host(backend, cfg, w, synth.FMT_Q4_K)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab_size, size=9)
    la = a.prefill(prompt, 0, want_logits=True)
    for pos, t in enumerate(prompt):
        lb, nb = b.forward_logits(pos, int(t))
    assert np.array_equal(la, lb)  # same kernels, same order: bit-identical
    ta = a.generate(nb, len(prompt), 20)
    tb, tok = [], nb
    for i in range(20):
        _, tok = b.forward_logits(len(prompt) + i, tok)
        tb.append(tok)
    assert list(ta) == tb
    assert a.launches_per_token() <= 5 * cfg.n_layers + 4


def test_model_argument_errors(backend):
    from slai_b200._lib import SlaiError
    from slai_b200.ops import GpuQuantMatrix
    cfg = Llama2Config(dim=256, hidden_dim=512, n_layers=1, n_q_heads=4, n_kv_heads=4, vocab_size=100, seq_len=16)
    from slai_b200.models import Llama2
    m = Llama2(backend, cfg)
    with pytest.raises(SlaiError):  # weights missing
        m.forward_logits(0, 1)
    bad = GpuQuantMatrix(backend, synth.FMT_Q4_K, 256, 512, synth.quantize(synth.FMT_Q4_K, synth.normal_matrix(1, 256, 512)))
    with pytest.raises(SlaiError) as e:
        m.set_matrix("wq", 0, bad)
    assert e.value.code == _lib.ERR_SHAPE
    w = synthetic_llama_host(cfg, synth.FMT_Q4_K, seed=1)
    m = llama_from_host(backend, cfg, w, synth.FMT_Q4_K)
    with pytest.raises(SlaiError):
        m.forward_logits(16, 1)  # pos == seq_len
    with pytest.raises(SlaiError):
        m.forward_logits(0, 100)  # token == vocab


@pytest.mark.parametrize("kv_dtype", [_lib.KV_F32, _lib.KV_F16])
def test_tiny_gpt2(backend, kv_dtype):
    p = Gpt2Params(**{**GPT2_TINY.__dict__, "kv_dtype": kv_dtype})
    w = synthetic_gpt2_host(p, seed=2, std=0.08, bias_std=0.05)
    m = gpt2_from_host(backend, p, w)
    ref = oracle_gpt2(p, w, kv_f16=(kv_dtype == _lib.KV_F16))
    rng = np.random.default_rng(3)
    tok = int(rng.integers(0, p.n_vocab))
    for pos in range(30):
        lg, nxt = m.forward(tok, pos)
        rl = ref.forward(tok, pos)
        assert rel_l2(lg, rl) < 1e-3, pos
        tok = O.argmax(rl)
    toks = m.generate(tok, 30, 10)
    assert len(toks) == 10


def test_gpt2_xl_shapes_one_layer(backend):
    """GPT-2 XL dimensions (E = 1600: an odd number of Q8_0 block pairs per row; vocab 50257 = 4*12564 + 1)."""
    p = Gpt2Params(n_vocab=50257, n_seq=32, n_embd=1600, n_head=25, n_layer=1, ff_len=6400, kv_dtype=_lib.KV_F32)
    w = synthetic_gpt2_host(p, seed=4, std=0.02, bias_std=0.02)
    m = gpt2_from_host(backend, p, w)
    ref = oracle_gpt2(p, w)
    tok = 50256
    for pos in range(3):
        lg, nxt = m.forward(tok, pos)
        rl = ref.forward(tok, pos)
        assert rel_l2(lg, rl) < 1e-3
        tok = O.argmax(rl)


def test_llama_stats_accounts_for_every_kernel_class(backend):
    """`slai_llama_stats`: one real decode step split by kernel class; the step leaves the same state as a plain one."""
    cfg = Llama2Config(dim=256, hidden_dim=512, n_layers=3, n_q_heads=4, n_kv_heads=2, vocab_size=500, seq_len=64)
    w = synthetic_llama_host(cfg, synth.FMT_Q4_K, seed=9, std=0.05, embd_std=1.0)
    a = llama_from_host(backend, cfg, w, synth.FMT_Q4_K)
    b = llama_from_host(backend, cfg, w, synth.FMT_Q4_K)
    for pos, tok in enumerate([3, 17, 42]):
        a.forward_logits(pos, tok)
        b.forward_logits(pos, tok)
    st = a.stats(7, 3)
    lg, nxt = b.forward_logits(3, 7)
    assert np.array_equal(a.read_state("logits"), lg)
    for name in ("qkv", "attention", "wo", "gate_up", "down"):
        assert st[name]["launches"] == cfg.n_layers and st[name]["us"] > 0, (name, st)
    assert st["logits"]["launches"] == 1 and st["logits"]["us"] > 0
    assert st["other"]["launches"] >= 1
    parts = sum(st[k]["us"] for k in ("other", "qkv", "attention", "wo", "gate_up", "down", "logits"))
    assert abs(parts - st["total_us"]) <= 1e-3 * st["total_us"] + 1.0
    lg2, _ = a.forward_logits(4, nxt)   # the graph path still works after a statistics step
    lg3, _ = b.forward_logits(4, nxt)
    assert np.array_equal(lg2, lg3)
