"""Several sequences decoded together (slai_llama_decode_batch): every sequence has its own KV cache and position, the weight
matrices are read once per step for all of them.  Per sequence: logits within 1e-3 relative L2 of the CPU oracle run on that
sequence alone and of the single-sequence decode step; greedy ids identical where the oracle's top two logits are apart."""
import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import synth, _lib
from slai_b200._lib import SlaiError
from slai_b200.models import TINY_LLAMA, Llama2Config, llama_from_host, synthetic_llama_host
from helpers import oracle_llama, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt,out_fmt,kv_dtype", [(synth.FMT_Q4_K, synth.FMT_Q6_K, _lib.KV_F16), (synth.FMT_Q8_0, synth.FMT_Q8_0, _lib.KV_F32),
                                                   (synth.FMT_Q5_K, synth.FMT_Q5_K, _lib.KV_F16)])
def test_batch_of_sequences_matches_each_alone(backend, fmt, out_fmt, kv_dtype):
    """Five sequences with different prompts; sequence b joins at step 2 b (so the positions inside a step differ) and one
    sequence leaves early.  Every step is checked against the oracle's own forward pass of that sequence."""
    cfg = Llama2Config(dim=512, hidden_dim=1280, n_layers=3, n_q_heads=8, n_kv_heads=2, vocab_size=2000, seq_len=64, kv_dtype=kv_dtype)
    w = synthetic_llama_host(cfg, fmt, out_fmt, seed=5, std=0.05, embd_std=1.0)
    m = llama_from_host(backend, cfg, w, fmt, out_fmt)
    B = 5
    m.batch_reserve(B)
    refs = [oracle_llama(cfg, w, fmt, out_fmt, kv_f16=(kv_dtype == _lib.KV_F16)) for _ in range(B)]
    rng = np.random.default_rng(1)
    prompts = rng.integers(0, cfg.vocab_size, size=(B, 6))
    tok = [int(prompts[b, 0]) for b in range(B)]
    pos = [-1] * B
    n_match = 0
    for step in range(24):
        active = [b for b in range(B) if step >= 2 * b and not (b == 1 and step >= 14)]   # sequence 1 stops after step 13
        for b in active:
            pos[b] += 1
        p = [pos[b] if b in active else -1 for b in range(B)]
        lg, nxt = m.decode_batch(tok, p)
        for b in active:
            rl = refs[b].forward(tok[b], pos[b])
            assert rel_l2(lg[b], rl) < 1e-3, (step, b)
            assert nxt[b] == int(np.argmax(lg[b]))
            if pos[b] + 1 < prompts.shape[1]:
                tok[b] = int(prompts[b, pos[b] + 1])
            else:
                top2 = np.partition(rl, -2)[-2:]
                if top2[1] - top2[0] > 1e-4 * np.abs(rl).max():
                    assert nxt[b] == O.argmax(rl), (step, b)
                    n_match += 1
                tok[b] = int(nxt[b])
    assert n_match > 20


def test_batch_equals_single_sequence_decode(backend):
    """The tiny-Llama benchmark configuration (dim 288: Q8_0 steps of 128 with a ragged last step): three sequences through the
    batch step against three models decoded one token at a time."""
    cfg = Llama2Config(**{**TINY_LLAMA.__dict__, "kv_dtype": _lib.KV_F32})
    w = synthetic_llama_host(cfg, synth.FMT_Q8_0, seed=9)
    mb = llama_from_host(backend, cfg, w, synth.FMT_Q8_0)
    mb.batch_reserve(3)
    singles = [llama_from_host(backend, cfg, w, synth.FMT_Q8_0) for _ in range(3)]
    tok = [11, 222, 3333]
    for pos in range(20):
        lg, nxt = mb.decode_batch(tok, [pos] * 3)
        for b in range(3):
            ls, ns = singles[b].forward_logits(pos, tok[b])
            assert rel_l2(lg[b], ls) < 1e-4, (pos, b)
            tok[b] = int(ns)
            top2 = np.partition(ls, -2)[-2:]
            if top2[1] - top2[0] > 1e-4 * np.abs(ls).max():
                assert nxt[b] == ns, (pos, b)
    # the single-sequence state of the batch model was never touched: it still decodes on its own cache
    l0, _ = mb.forward_logits(0, 11)
    l1, _ = llama_from_host(backend, cfg, w, synth.FMT_Q8_0).forward_logits(0, 11)
    assert np.array_equal(l0.view(np.uint32), l1.view(np.uint32))


def test_batch_step_across_a_graph_boundary(backend):
    """The replayed step is captured again when the longest context crosses a multiple of 256 positions: two sequences, one
    256 positions ahead of... the other never leaving the first bucket, decoded past position 256."""
    cfg = Llama2Config(dim=256, hidden_dim=512, n_layers=2, n_q_heads=4, n_kv_heads=2, vocab_size=1000, seq_len=320, kv_dtype=_lib.KV_F16)
    w = synthetic_llama_host(cfg, synth.FMT_Q4_K, synth.FMT_Q6_K, seed=2, std=0.05, embd_std=1.0)
    mb = llama_from_host(backend, cfg, w, synth.FMT_Q4_K, synth.FMT_Q6_K)
    mb.batch_reserve(2)
    singles = [llama_from_host(backend, cfg, w, synth.FMT_Q4_K, synth.FMT_Q6_K) for _ in range(2)]
    tok = [5, 77]
    for step in range(266):
        pos = [step, step // 2]     # sequence 1 advances every other step and stays below 256
        p = [pos[0], pos[1] if step % 2 == 0 else -1]
        lg, nxt = mb.decode_batch(tok, p)
        for b in range(2):
            if p[b] < 0:
                continue
            ls, ns = singles[b].forward_logits(p[b], tok[b])
            if step < 4 or step > 250:
                assert rel_l2(lg[b], ls) < 1e-4, (step, b)
            tok[b] = int(ns)


def test_batch_argument_errors(backend):
    cfg = Llama2Config(**{**TINY_LLAMA.__dict__, "kv_dtype": _lib.KV_F32})
    m = llama_from_host(backend, cfg, synthetic_llama_host(cfg, synth.FMT_Q8_0, seed=9), synth.FMT_Q8_0)
    with pytest.raises(SlaiError) as e:   # nothing reserved
        m.decode_batch([1, 2], [0, 0])
    assert e.value.code == _lib.ERR_INVALID_ARG
    with pytest.raises(SlaiError):
        m.batch_reserve(9)
    m.batch_reserve(2)
    with pytest.raises(SlaiError):
        m.decode_batch([1, 2, 3], [0, 0, 0])
    with pytest.raises(SlaiError):
        m.decode_batch([1, cfg.vocab_size], [0, 0])
    with pytest.raises(SlaiError):
        m.decode_batch([1, 2], [0, cfg.seq_len])
    lg, nxt = m.decode_batch([1, 2], [0, -1])   # a sequence left out
    assert np.isfinite(lg[0]).all() and nxt[0] == int(np.argmax(lg[0]))
    lg1, _ = m.decode_batch([1], [0])           # fewer sequences than reserved; one sequence takes the single-vector kernels
    l0, _ = m.forward_logits(0, 1)
    assert rel_l2(lg1[0], l0) < 1e-4 and rel_l2(lg[0], l0) < 1e-4
    m.batch_reserve(0)
    with pytest.raises(SlaiError):
        m.decode_batch([1], [0])
