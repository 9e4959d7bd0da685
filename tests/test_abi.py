"""The C-ABI library builds, loads and exports every function the header declares (no compute without a GPU)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    src = open(os.path.join(ROOT, "include", "slai_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(slai_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def lib():
    from slai_b200 import build, _lib
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    from slai_b200 import _lib
    names = header_functions()
    assert len(names) >= 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(_lib.SIGNATURES) == names  # the Python binding covers exactly the header


def test_rust_binding_source_covers_the_header():
    rs = open(os.path.join(ROOT, "rust", "slai-b200-sys", "src", "lib.rs")).read()
    missing = [n for n in header_functions() if f"pub fn {n}(" not in rs]
    assert not missing, missing


def test_safe_rust_wrapper_calls_only_declared_functions_and_mirrors_the_operators():
    """The safe crate (rust/slai-b200) is source only: check what can be checked without a Rust toolchain.  Every
    `sys::slai_*` it calls is declared in the -sys crate with the same number of arguments, and the reference's operator
    types each have a `launch`."""
    import re
    sysrs = open(os.path.join(ROOT, "rust", "slai-b200-sys", "src", "lib.rs")).read()
    decl = {m.group(1): m.group(2) for m in re.finditer(r"pub fn (slai_\w+)\(([^)]*)\)", sysrs)}
    src = ""
    for f in ("lib.rs", "ops.rs", "models.rs"):
        src += open(os.path.join(ROOT, "rust", "slai-b200", "src", f)).read()
    calls = re.findall(r"sys::(slai_\w+)\(", src)
    assert len(set(calls)) >= 35
    for name in set(calls):
        assert name in decl, name
    # argument counts: split the call's argument text at top-level commas
    for m in re.finditer(r"sys::(slai_\w+)\(", src):
        i, depth, args, cur = m.end(), 1, [], ""
        while depth:
            ch = src[i]
            if ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
                if depth == 0:
                    break
            if ch == "," and depth == 1:
                args.append(cur)
                cur = ""
            else:
                cur += ch
            i += 1
        if cur.strip():
            args.append(cur)
        want = len([a for a in decl[m.group(1)].split(",") if a.strip()])
        assert len(args) == want, (m.group(1), len(args), want)
    for op in ("GemvQuant", "RmsNorm", "RoPE", "Silu", "Unary", "BatchedMultiqueryAttention"):
        assert re.search(r"impl " + op + r" \{.*?pub fn launch", src, re.S), op
    for op in ("SoftMax", "LayerNorm"):
        assert re.search(r"impl " + op + r" \{.*?pub fn launch_cols", src, re.S), op
    for name in ("matmul_quant_assign", "add_assign", "mul_assign", "copy", "begin_submission", "submit", "forward_logits"):
        assert f"pub fn {name}" in src, name


def test_header_cites_reference_interfaces():
    src = open(os.path.join(ROOT, "include", "slai_b200.h")).read()
    for cite in ("gemv_quant.rs:206-312", "rms_norm.rs:35-67", "rope.rs:45-85", "silu.rs:24-48", "softmax.rs:22-40",
                 "layernorm.rs:25-60", "batched_multiquery_attention.rs:32-100", "transformer.rs:316-381", "gguf.rs:133-194"):
        assert cite in src, cite


def test_no_cpu_fallback(lib):
    """Without a CUDA device the library refuses to create a context (it never computes on the host)."""
    if lib.slai_device_count() > 0:
        pytest.skip("a GPU is visible")
    h = C.c_void_p()
    rc = lib.slai_ctx_create(0, C.byref(h))
    assert rc == 4 and not h.value  # SLAI_ERR_CUDA
    assert b"no CPU fallback" in lib.slai_last_error_string(None)
    from slai_b200._lib import SlaiError
    from slai_b200.ops import Backend
    with pytest.raises(SlaiError):
        Backend(0)


def test_null_arguments_are_rejected(lib):
    assert lib.slai_ctx_create(0, None) == 1
    assert lib.slai_ctx_sync(None) == 1
    assert lib.slai_gemv_quant(None, None, None, None, 1) == 1
    assert lib.slai_llama_decode(None, 0, 0, None, None) == 1
    assert lib.slai_qmatrix_destroy(None) == 0 and lib.slai_ctx_destroy(None) == 0


def test_algorithmic_byte_table():
    """GEMV bytes = M*K*bpw/8 + 4K + 4M for the benchmark shapes."""
    from slai_b200 import synth
    assert synth.gemv_bytes(synth.FMT_Q4_K, 4096, 4096) == 9_469_952
    assert synth.gemv_bytes(synth.FMT_Q8_0, 4096, 4096) == 17_858_560
    assert synth.gemv_bytes(synth.FMT_Q6_K, 32000, 4096) == 107_664_384
    assert synth.gemv_bytes(synth.FMT_Q5_K, 11008, 4096) == 31_058_944
    from slai_b200.models import LLAMA2_7B, LLAMA2_70B, GPT2_XL
    assert LLAMA2_7B.weight_bytes_per_token(synth.FMT_Q4_K, synth.FMT_Q6_K) == 3_750_273_024
    assert LLAMA2_70B.weight_bytes_per_token(synth.FMT_Q4_K, synth.FMT_Q6_K) == 38_718_750_720
    assert GPT2_XL.weight_bytes_per_token(synth.FMT_Q8_0) == 1_652_156_900
    assert LLAMA2_7B.kv_bytes_at(0) == 524_288
