"""Shared helpers of the test-suite: oracle models built from the same host weights as the CUDA models."""
import numpy as np

from oracle import oracle as O
from slai_b200 import synth


def rel_l2(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def oracle_llama(cfg, weights, fmt, out_fmt=None, kv_f16=False, nthreads=8):
    out_fmt = fmt if out_fmt is None else out_fmt
    m = O.Llama(dim=cfg.dim, hidden=cfg.hidden_dim, n_layers=cfg.n_layers, n_q=cfg.n_q_heads, n_kv=cfg.n_kv_heads,
                vocab=cfg.vocab_size, seq_len=cfg.seq_len, rope_base=cfg.rope_base_freq, eps=cfg.rms_norm_eps,
                neox=bool(cfg.rope_variant), kv_f16=kv_f16, nthreads=nthreads)
    shapes = cfg.matrix_shapes()
    for (name, l), val in weights.items():
        if name in shapes:
            m.set_weight(name, l, O.dequantize(fmt, val).reshape(shapes[name]))
        elif name == "output":
            m.set_weight(name, l, O.dequantize(out_fmt, val).reshape(cfg.vocab_size, cfg.dim))
        else:
            m.set_weight(name, l, val)
    return m


def oracle_gpt2(p, weights, fmt=synth.FMT_Q8_0, kv_f16=False, nthreads=8):
    m = O.Gpt2(n_vocab=p.n_vocab, n_seq=p.n_seq, n_embd=p.n_embd, n_head=p.n_head, n_layer=p.n_layer, ff_len=p.ff_len,
               eps=p.layernorm_eps, kv_f16=kv_f16, nthreads=nthreads)
    shapes = p.matrix_shapes()
    for (name, l), val in weights.items():
        if name in shapes:
            m.set_weight(name, l, O.dequantize(fmt, val).reshape(shapes[name]))
        elif name == "wte":
            m.set_weight(name, l, O.dequantize(fmt, val).reshape(p.n_vocab, p.n_embd))
        else:
            m.set_weight(name, l, val)
    return m
