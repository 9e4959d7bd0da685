"""The dequant-GEMV kernel's per-lane code (fragment mapping, load offsets, scale handling) executed on the CPU:
32 host threads play a warp with an emulated m16n8k16 MMA (tests/host_emul.cpp), checked against the oracle."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INC = "/usr/local/cuda/include"


@pytest.fixture(scope="module")
def emul(tmp_path_factory):
    if not os.path.exists(os.path.join(CUDA_INC, "cuda_fp16.h")) or shutil.which("g++") is None:
        pytest.skip("CUDA headers or g++ not available")
    exe = str(tmp_path_factory.mktemp("emul") / "host_emul")
    subprocess.check_call(["g++", "-std=c++17", "-O1", f"-I{CUDA_INC}", "-o", exe, os.path.join(ROOT, "tests", "host_emul.cpp"), "-lpthread"])
    return exe


CASES = [(synth.FMT_Q4_K, 256), (synth.FMT_Q4_K, 2816), (synth.FMT_Q5_K, 512), (synth.FMT_Q5_K, 2816), (synth.FMT_Q6_K, 256),
         (synth.FMT_Q6_K, 2816), (synth.FMT_Q8_0, 32), (synth.FMT_Q8_0, 288), (synth.FMT_Q8_0, 1600)]


@pytest.mark.parametrize("fmt,K", CASES)
@pytest.mark.parametrize("kind", ["quantized", "random_bits"])
def test_emulated_warp_matches_oracle(emul, tmp_path, fmt, K, kind):
    rng = np.random.default_rng(K + fmt)
    blocks = synth.quantize(fmt, synth.normal_matrix(K, 16, K)) if kind == "quantized" else synth.random_blocks(fmt, 16, K, rng)
    v = (rng.standard_normal(K) * (1e-3 if kind == "quantized" else 3.0)).astype(np.float32)
    blocks.tofile(tmp_path / "b.bin")
    v.tofile(tmp_path / "v.bin")
    out = subprocess.run([emul, str(fmt), str(K), str(tmp_path / "b.bin"), str(tmp_path / "v.bin")], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    got = np.array([float(t) for t in out.stdout.split()], dtype=np.float32)
    ref = O.dequantize(fmt, blocks).reshape(16, K).astype(np.float64) @ v.astype(np.float64)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 2e-6


BATCH_CASES = [(synth.FMT_Q4_K, 512, 8), (synth.FMT_Q4_K, 2816, 4), (synth.FMT_Q5_K, 768, 8), (synth.FMT_Q5_K, 256, 2), (synth.FMT_Q6_K, 512, 8),
               (synth.FMT_Q6_K, 2816, 2), (synth.FMT_Q8_0, 288, 8), (synth.FMT_Q8_0, 1600, 4)]


@pytest.mark.parametrize("fmt,K,nv", BATCH_CASES)
@pytest.mark.parametrize("kind", ["quantized", "random_bits"])
def test_emulated_warp_batched_matches_oracle(emul, tmp_path, fmt, K, nv, kind):
    """The batched per-lane code (one pass over the packed weights for several vectors, each with its own scale)."""
    rng = np.random.default_rng(K + fmt + nv)
    blocks = synth.quantize(fmt, synth.normal_matrix(K, 16, K)) if kind == "quantized" else synth.random_blocks(fmt, 16, K, rng)
    v = (rng.standard_normal((nv, K)) * np.logspace(-3, 1, nv)[:, None]).astype(np.float32)
    v[nv - 1] = 0.0  # a zero vector among them
    blocks.tofile(tmp_path / "b.bin")
    v.tofile(tmp_path / "v.bin")
    out = subprocess.run([emul, str(fmt), str(K), str(tmp_path / "b.bin"), str(tmp_path / "v.bin"), str(nv)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    got = np.array([float(t) for t in out.stdout.split()], dtype=np.float32).reshape(nv, 16)
    ref = v.astype(np.float64) @ O.dequantize(fmt, blocks).reshape(16, K).astype(np.float64).T
    assert np.all(got[nv - 1] == 0.0)
    for i in range(nv - 1):
        assert np.linalg.norm(got[i] - ref[i]) / np.linalg.norm(ref[i]) < 2e-6
