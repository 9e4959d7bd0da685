"""GGUF reader: files written by a minimal writer (and, when the `gguf` python package is importable, by its
GGUFWriter) parse to the same metadata and tensor bytes; a model built from a file decodes like the oracle."""
import os
import struct

import numpy as np
import pytest

from slai_b200 import gguf_io, synth
from slai_b200.models import Llama2Config, synthetic_llama_host

NAMES = dict(wq="attn_q.weight", wk="attn_k.weight", wv="attn_v.weight", wo="attn_output.weight", w_gate="ffn_gate.weight",
             w_up="ffn_up.weight", w_down="ffn_down.weight", attn_norm="attn_norm.weight", ffn_norm="ffn_norm.weight")


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, metadata: dict, tensors: list, alignment: int = 32, version: int = 3):
    """tensors: (name, dims (cols first), ggml type, bytes)."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(metadata)))
    for k, v in metadata.items():
        out += _s(k)
        if isinstance(v, bool):
            out += struct.pack("<I?", 7, v)
        elif isinstance(v, int):
            out += struct.pack("<II", 4, v)
        elif isinstance(v, float):
            out += struct.pack("<If", 6, v)
        elif isinstance(v, str):
            out += struct.pack("<I", 8) + _s(v)
        elif isinstance(v, list) and all(isinstance(i, str) for i in v):
            out += struct.pack("<IIQ", 9, 8, len(v)) + b"".join(_s(i) for i in v)
        elif isinstance(v, np.ndarray) and v.dtype == np.float32:
            out += struct.pack("<IIQ", 9, 6, v.size) + v.tobytes()
        else:
            raise TypeError(k)
    off, offsets = 0, []
    for _, _, _, data in tensors:
        offsets.append(off)
        off = (off + len(data) + alignment - 1) // alignment * alignment
    for (name, dims, gt, _), o in zip(tensors, offsets):
        out += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", gt, o)
    out += b"\0" * ((-len(out)) % alignment)
    for (_, _, _, data), o in zip(tensors, offsets):
        assert len(out) % alignment == 0
        out += bytes(data) + b"\0" * ((-len(data)) % alignment)
    with open(path, "wb") as f:
        f.write(out)


def tiny_model_file(path, fmt=synth.FMT_Q8_0, tied=False, alignment=32):
    cfg = Llama2Config(dim=256, hidden_dim=512, n_layers=2, n_q_heads=4, n_kv_heads=2, vocab_size=300, seq_len=40, rope_base_freq=5000.0,
                       rms_norm_eps=1e-5)
    w = synthetic_llama_host(cfg, fmt, seed=9, std=0.05, embd_std=1.0)
    md = {"general.architecture": "llama", "general.alignment": alignment, "llama.embedding_length": cfg.dim,
          "llama.feed_forward_length": cfg.hidden_dim, "llama.block_count": cfg.n_layers, "llama.attention.head_count": cfg.n_q_heads,
          "llama.attention.head_count_kv": cfg.n_kv_heads, "llama.context_length": cfg.seq_len, "llama.rope.freq_base": cfg.rope_base_freq,
          "llama.attention.layer_norm_rms_epsilon": cfg.rms_norm_eps, "tokenizer.ggml.tokens": [f"t{i}" for i in range(cfg.vocab_size)],
          "tokenizer.ggml.scores": np.zeros(cfg.vocab_size, dtype=np.float32), "some.flag": True}
    shapes = cfg.matrix_shapes()
    tensors = []
    for (name, l), val in w.items():
        if name in shapes:
            r, c = shapes[name]
            tensors.append((f"blk.{l}.{NAMES[name]}", (c, r), fmt, np.asarray(val, np.uint8).tobytes()))
        elif name in ("attn_norm", "ffn_norm"):
            tensors.append((f"blk.{l}.{NAMES[name]}", (cfg.dim,), 0, np.asarray(val, np.float32).tobytes()))
    tensors.append(("token_embd.weight", (cfg.dim, cfg.vocab_size), 1, w[("token_embd", -1)].astype(np.float16).tobytes()))
    tensors.append(("output_norm.weight", (cfg.dim,), 0, w[("out_norm", -1)].tobytes()))
    if not tied:
        tensors.append(("output.weight", (cfg.dim, cfg.vocab_size), fmt, np.asarray(w[("output", -1)], np.uint8).tobytes()))
    write_gguf(path, md, tensors, alignment)
    w[("token_embd", -1)] = w[("token_embd", -1)].astype(np.float16).astype(np.float32)  # what the file holds
    return cfg, w


@pytest.mark.parametrize("alignment", [32, 64])
def test_reader_round_trip(tmp_path, alignment):
    path = str(tmp_path / "m.gguf")
    cfg, w = tiny_model_file(path, alignment=alignment)
    g = gguf_io.GgufFile(path)
    assert g.version == 3 and g.metadata["general.architecture"] == "llama" and g.metadata["some.flag"] is True
    assert len(g.metadata["tokenizer.ggml.tokens"]) == cfg.vocab_size and g.metadata["tokenizer.ggml.tokens"][7] == "t7"
    assert g.metadata["tokenizer.ggml.scores"].dtype == np.float32 and g.metadata["tokenizer.ggml.scores"].size == cfg.vocab_size
    got = gguf_io.llama_config_from_gguf(g)
    assert (got.dim, got.hidden_dim, got.n_layers, got.n_q_heads, got.n_kv_heads, got.vocab_size, got.seq_len) == \
           (cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_q_heads, cfg.n_kv_heads, cfg.vocab_size, cfg.seq_len)
    assert got.rope_base_freq == 5000.0 and abs(got.rms_norm_eps - 1e-5) < 1e-12
    t = g.tensors["blk.1.ffn_down.weight"]
    assert (t.rows, t.cols, t.ggml_type) == (cfg.dim, cfg.hidden_dim, synth.FMT_Q8_0)
    assert np.array_equal(t.data, np.asarray(w[("w_down", 1)], np.uint8).reshape(-1))
    assert np.array_equal(g.tensors["token_embd.weight"].to_f32().reshape(cfg.vocab_size, cfg.dim), w[("token_embd", -1)])
    g.close()


def test_reader_defaults_and_errors(tmp_path):
    p = str(tmp_path / "x.gguf")
    write_gguf(p, {"llama.embedding_length": 64, "llama.feed_forward_length": 128, "llama.block_count": 1, "llama.attention.head_count": 2,
                   "llama.attention.head_count_kv": 2, "llama.context_length": 16, "tokenizer.ggml.tokens": ["a", "b"]}, [])
    c = gguf_io.llama_config_from_gguf(gguf_io.GgufFile(p))
    assert c.rope_base_freq == 10000.0 and c.rms_norm_eps == 1.0e-6 and c.vocab_size == 2   # the reference's defaults
    with open(p, "wb") as f:
        f.write(b"GGML" + b"\0" * 32)
    with pytest.raises(gguf_io.GgufError):
        gguf_io.GgufFile(p)
    write_gguf(p, {}, [("t", (64, 2), 8, b"\0" * 10)])  # data shorter than the header promises
    with pytest.raises(gguf_io.GgufError):
        gguf_io.GgufFile(p)
    write_gguf(p, {}, [], version=1)
    with pytest.raises(gguf_io.GgufError):
        gguf_io.GgufFile(p)


def test_agrees_with_the_gguf_package(tmp_path):
    gguf = pytest.importorskip("gguf")
    # a file written by the package's writer parses identically with this reader ...
    p = str(tmp_path / "pkg.gguf")
    wr = gguf.GGUFWriter(p, "llama")
    wr.add_uint32("llama.block_count", 3)
    wr.add_float32("llama.rope.freq_base", 12345.0)
    wr.add_array("tokenizer.ggml.tokens", ["x", "yy", "zzz"])
    a = np.arange(64 * 4, dtype=np.float32).reshape(4, 64)
    blocks = synth.quantize(synth.FMT_Q8_0, a)
    wr.add_tensor("dense", a)
    wr.add_tensor("quant", np.asarray(blocks, np.uint8).reshape(4, -1), raw_dtype=gguf.GGMLQuantizationType.Q8_0)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    g = gguf_io.GgufFile(p)
    assert g.metadata["llama.block_count"] == 3 and g.metadata["llama.rope.freq_base"] == 12345.0
    assert list(g.metadata["tokenizer.ggml.tokens"]) == ["x", "yy", "zzz"]
    assert (g.tensors["dense"].rows, g.tensors["dense"].cols) == (4, 64)
    assert np.array_equal(g.tensors["dense"].to_f32().reshape(4, 64), a)
    assert g.tensors["quant"].ggml_type == synth.FMT_Q8_0 and (g.tensors["quant"].rows, g.tensors["quant"].cols) == (4, 64)
    assert np.array_equal(g.tensors["quant"].data, np.asarray(blocks, np.uint8).reshape(-1))
    # ... and a file from the minimal writer parses identically with the package's reader
    p2 = str(tmp_path / "m.gguf")
    cfg, w = tiny_model_file(p2)
    rd = gguf.GGUFReader(p2)
    t = {x.name: x for x in rd.tensors}
    mine = gguf_io.GgufFile(p2)
    for name in ("blk.0.attn_q.weight", "blk.1.ffn_down.weight", "output_norm.weight"):
        assert np.array_equal(np.asarray(t[name].data).view(np.uint8).reshape(-1), mine.tensors[name].data)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,tied", [(synth.FMT_Q8_0, False), (synth.FMT_Q4_K, True)])
def test_model_from_gguf_matches_oracle(backend, tmp_path, fmt, tied):
    from helpers import oracle_llama, rel_l2
    from oracle import oracle as O
    from slai_b200 import _lib
    path = str(tmp_path / "m.gguf")
    cfg, w = tiny_model_file(path, fmt=fmt, tied=tied)
    cfg.kv_dtype = _lib.KV_F32
    g = gguf_io.GgufFile(path)
    m = gguf_io.llama_from_gguf(backend, g, kv_dtype=_lib.KV_F32)
    if tied:
        w[("output", -1)] = None
    ref = oracle_llama(cfg, {k: v for k, v in w.items() if v is not None}, fmt)
    if tied:  # the oracle ties the output matrix to the f32 embedding
        ref.set_weight("output", -1, w[("token_embd", -1)].reshape(cfg.vocab_size, cfg.dim))
    tok = 5
    for pos in range(6):
        lg, nxt = m.forward_logits(pos, tok)
        rl = ref.forward(tok, pos)
        assert rel_l2(lg, rl) < 1e-3, pos
        tok = O.argmax(rl)


def test_reference_parse_fixture():
    """The reference's own parse fixture (assets/gguf/dummy.gguf, copied to tests/golden/): version 3, fifteen metadata
    entries covering every scalar type, strings and arrays, ten f32 tensors; read by this repository's reader and, when
    it is importable, identically by the `gguf` python package."""
    path = os.path.join(os.path.dirname(__file__), "golden", "dummy.gguf")
    g = gguf_io.GgufFile(path)
    assert g.version == 3 and len(g.metadata) == 15 and len(g.tensors) == 10
    md = g.metadata
    assert md["some.parameter.uint8"] == 0x12 and md["some.parameter.int8"] == -0x13
    assert md["some.parameter.uint16"] == 0x1234 and md["some.parameter.int16"] == -0x1235
    assert md["some.parameter.uint32"] == 0x12345678 and md["some.parameter.int32"] == -0x12345679
    assert md["some.parameter.uint64"] == 0x123456789ABCDEF0 and md["some.parameter.int64"] == -0x123456789ABCDEF1
    assert abs(md["some.parameter.float32"] - 0.123456789) < 1e-7 and abs(md["some.parameter.float64"] - 0.1234567890123456789) < 1e-15
    assert md["some.parameter.bool"] is True and md["some.parameter.string"] == "hello world"
    assert len(md["some.parameter.arr.i16"]) == 4 and len(md["some.parameter.arr.f32"]) == 3 and len(md["some.parameter.arr.str"]) == 3
    for t in g.tensors.values():
        assert t.ggml_type == 0 and t.data.size == 4 * int(np.prod(t.dims))
    try:
        from gguf import GGUFReader
    except Exception:
        g.close()
        return
    r = GGUFReader(path)
    theirs = {t.name: t for t in r.tensors}
    assert sorted(theirs) == sorted(g.tensors)
    for name, t in g.tensors.items():
        assert np.array_equal(np.frombuffer(bytes(t.data), dtype=np.uint8), np.asarray(theirs[name].data).view(np.uint8).reshape(-1))
    g.close()
