"""Generates the committed fixtures under tests/golden/.  Run from the repository root:

    python tests/golden/make_golden.py

1. block_recipes.npz — the deterministic blocks of the reference's (disabled) dequantisation test
   (crates/slai/src/ops/quantization.rs:77-221: Q8_0 `scale=f16(1.234), data[k]=i*16-128+k`; Q4_K/Q5_K
   `d=f16(1.234), dmin=f16(5.678), scales[k]=16i+k, qs/qh[k]=sat(16i+k)`; Q6_K `scales[k]=8i-127+k,
   ql/qh[k]=8i+k, d bits=123`) with the values `Block*::dequantize()` yields for them, computed by the CPU
   oracle and — when the `gguf` python package is importable — required to equal its independent
   dequantiser bit for bit before being written.
2. tiny_llama_greedy.npz — the tiny-Llama benchmark configuration (tiny Llama-2 architecture, Q8_0, 16-token seeded prompt, 128
   greedy tokens) run through the CPU oracle: prompt, generated ids and the top-1/top-2 logit margin per step.

The reference itself cannot be run here (Rust, no toolchain), so these are oracle outputs pinned against
the reference's recipes, not outputs of the reference binary.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from slai_b200 import synth  # noqa: E402
from slai_b200.models import TINY_LLAMA, synthetic_llama_host  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def f16_bits(x):
    return int(np.array([x], dtype=np.float32).astype(np.float16).view(np.uint16)[0])


def sat_u8(a):
    return np.minimum(a, 255).astype(np.uint8)


def recipes():
    out = {}
    # Q8_0: 8 blocks
    b = np.zeros((8, 34), dtype=np.uint8)
    for i in range(8):
        b[i, 0:2] = np.array([f16_bits(1.234)], dtype=np.uint16).view(np.uint8)
        data = ((i * 16 - 128) + np.arange(32)).astype(np.int64)
        b[i, 2:] = ((data + 128) % 256 - 128).astype(np.int8).view(np.uint8)  # i8 wrapping add
    out[synth.FMT_Q8_0] = b
    # Q4_K / Q5_K: 16 blocks
    for fmt, size in ((synth.FMT_Q4_K, 144), (synth.FMT_Q5_K, 176)):
        b = np.zeros((16, size), dtype=np.uint8)
        for i in range(16):
            b[i, 0:2] = np.array([f16_bits(1.234)], dtype=np.uint16).view(np.uint8)
            b[i, 2:4] = np.array([f16_bits(5.678)], dtype=np.uint16).view(np.uint8)
            b[i, 4:16] = ((i * 16 + np.arange(12)) % 256).astype(np.uint8)
            qs = sat_u8(i * 16 + np.arange(128))
            qh = sat_u8(i * 16 + np.arange(32))
            if fmt == synth.FMT_Q4_K:
                b[i, 16:] = qs
            else:
                b[i, 16:48] = qh
                b[i, 48:] = qs
        out[fmt] = b
    # Q6_K: 16 blocks
    b = np.zeros((16, 210), dtype=np.uint8)
    for i in range(16):
        b[i, 0:128] = ((i * 8 + np.arange(128)) % 256).astype(np.uint8)
        b[i, 128:192] = ((i * 8 + np.arange(64)) % 256).astype(np.uint8)
        sc = (i * 8 - 127) + np.arange(16)
        b[i, 192:208] = ((sc + 128) % 256 - 128).astype(np.int8).view(np.uint8)
        b[i, 208:210] = np.array([123], dtype=np.uint16).view(np.uint8)
    out[synth.FMT_Q6_K] = b
    # legacy formats (ops/quantization.rs:85-148): 16 blocks each, qs[k] = 16 i + k, d = f16(1.234); Q4_1 m = raw bits 3,
    # Q5_x qh = [1, 100, 200, 250], Q5_1 m = raw bits 125; Q8_K d = 1.234f, qs[k] = saturating (8 i - 127) + (k as i8), bsums 0
    half = np.array([1.234], dtype=np.float32).astype(np.float16).view(np.uint8)
    qh = np.array([1, 100, 200, 250], dtype=np.uint8)
    for fmt, hdr in ((synth.FMT_Q4_0, [half]), (synth.FMT_Q4_1, [half, np.array([3], np.uint16).view(np.uint8)]),
                     (synth.FMT_Q5_0, [half, qh]), (synth.FMT_Q5_1, [half, np.array([125], np.uint16).view(np.uint8), qh])):
        b = np.zeros((16, synth.BLOCK_BYTES[fmt]), dtype=np.uint8)
        h = np.concatenate(hdr)
        for i in range(16):
            b[i, :h.size] = h
            b[i, h.size:] = (16 * i + np.arange(16)).astype(np.uint8)
        out[fmt] = b
    b = np.zeros((16, 292), dtype=np.uint8)
    for i in range(16):
        b[i, 0:4] = np.array([1.234], dtype=np.float32).view(np.uint8)
        k = np.arange(256).astype(np.uint8).view(np.int8).astype(np.int32)
        b[i, 4:260] = np.clip(8 * i - 127 + k, -128, 127).astype(np.int8).view(np.uint8)
    out[synth.FMT_Q8_K] = b
    return out


def main():
    rec = recipes()
    save = {}
    try:
        from gguf import quants, GGMLQuantizationType as T
        tmap = {synth.FMT_Q8_0: T.Q8_0, synth.FMT_Q4_K: T.Q4_K, synth.FMT_Q5_K: T.Q5_K, synth.FMT_Q6_K: T.Q6_K, synth.FMT_Q4_0: T.Q4_0,
                synth.FMT_Q4_1: T.Q4_1, synth.FMT_Q5_0: T.Q5_0, synth.FMT_Q5_1: T.Q5_1}
    except Exception:  # pragma: no cover
        quants, tmap = None, {}
    for fmt, blocks in rec.items():
        vals = O.dequantize(fmt, blocks)
        if quants is not None and fmt in tmap:
            ref = quants.dequantize(blocks, tmap[fmt]).reshape(-1)
            assert np.array_equal(vals.view(np.uint32), ref.astype(np.float32).view(np.uint32)), synth.FMT_NAMES[fmt]
        name = synth.FMT_NAMES[fmt]
        save[f"{name}_blocks"] = blocks
        save[f"{name}_values"] = vals
    np.savez_compressed(os.path.join(HERE, "block_recipes.npz"), **save)
    print("block_recipes.npz written; cross-checked with gguf:", quants is not None)

    cfg = TINY_LLAMA
    # seed 4: among seeds 1..8 the one whose top-1/top-2 logit margin over the first 64 greedy steps is largest
    # (1.4e-3; logits are nearly flat with N(0,0.02) weights, so small margins would make greedy ids fragile)
    w = synthetic_llama_host(cfg, synth.FMT_Q8_0, seed=4)
    model = O.Llama(dim=cfg.dim, hidden=cfg.hidden_dim, n_layers=cfg.n_layers, n_q=cfg.n_q_heads, n_kv=cfg.n_kv_heads,
                    vocab=cfg.vocab_size, seq_len=cfg.seq_len, eps=cfg.rms_norm_eps, nthreads=8)
    shapes = cfg.matrix_shapes()
    for (name, l), val in w.items():
        if name in shapes:
            r, c = shapes[name]
            model.set_weight(name, l, O.dequantize(synth.FMT_Q8_0, val).reshape(r, c))
        elif name == "output":
            model.set_weight(name, l, O.dequantize(synth.FMT_Q8_0, val).reshape(cfg.vocab_size, cfg.dim))
        else:
            model.set_weight(name, l, val)
    prompt = np.random.default_rng(1234).integers(0, cfg.vocab_size, size=16).astype(np.int32)
    toks, margins = [], []
    tok = int(prompt[0])
    for pos in range(16 + 128 - 1):
        logits = model.forward(tok, pos)
        if pos + 1 < 16:
            tok = int(prompt[pos + 1])  # forced (crates/slai-chat/src/sampler.rs:102-107)
        else:
            tok = O.argmax(logits)
            top2 = np.partition(logits, -2)[-2:]
            toks.append(tok)
            margins.append(float(top2[1] - top2[0]))
    np.savez_compressed(os.path.join(HERE, "tiny_llama_greedy.npz"), prompt=prompt, tokens=np.array(toks, dtype=np.int32),
                        margins=np.array(margins, dtype=np.float32), seed=np.array([4]))
    print("tiny_llama_greedy.npz written:", toks[:16], "min margin", min(margins))


if __name__ == "__main__":
    main()
