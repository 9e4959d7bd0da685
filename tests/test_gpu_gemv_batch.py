"""A batch of input vectors in one pass over a quantised matrix (slai_gemv_quant with n_batch > 1), through the C ABI,
against the CPU oracle's dequantised weights and against the single-vector kernel.  Tolerance as for the GEMV: <= 1e-3
relative L2 per vector (measured far inside)."""
import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import synth
from slai_b200.ops import GpuQuantMatrix
from helpers import rel_l2

pytestmark = pytest.mark.gpu
FMTS = [synth.FMT_Q8_0, synth.FMT_Q4_K, synth.FMT_Q5_K, synth.FMT_Q6_K]


def run_batch(backend, ctx, m, v):
    nb, _ = v.shape
    out = backend.zeros(nb * m.nrows)
    ctx.matmul_quant_assign(out, m, backend.vector(v), n_batch=nb)
    return out.to_numpy().reshape(nb, m.nrows)


# ragged row counts, one and many chunks of K, the benchmark's widths, the 70B feed-forward width
SHAPES = [(16, 256), (5, 512), (300, 2816), (1000, 4096), (4096, 4096), (512, 11008), (272, 28672)]


# all shapes with a full batch; the smaller instantiations (2 and 4 vectors, partly filled) on two of them
CASES = [(s, 8) for s in SHAPES] + [(s, nb) for s in ((300, 2816), (1000, 4096)) for nb in (2, 3, 5)]


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("shape,nb", CASES)
def test_gemv_batch_parity(backend, ctx, fmt, shape, nb):
    M, K = shape
    rng = np.random.default_rng(M + 31 * K + fmt + nb)
    blocks = synth.quantize(fmt, synth.normal_matrix(M * 7 + K, M, K))
    v = rng.standard_normal((nb, K)).astype(np.float32)
    m = GpuQuantMatrix(backend, fmt, M, K, blocks)
    got = run_batch(backend, ctx, m, v)
    w = O.dequantize(fmt, blocks).reshape(M, K).astype(np.float64)
    for b in range(nb):
        assert rel_l2(got[b], w @ v[b].astype(np.float64)) < 1e-5
    # the oracle's own f32 GEMV on one of the vectors, and the single-vector kernel on all of them
    assert rel_l2(got[nb - 1], O.gemv_quant(fmt, blocks, v[nb - 1], M, K, nthreads=8)) < 1e-3
    if K == 28672 and fmt in (synth.FMT_Q5_K, synth.FMT_Q6_K):
        return  # the single-vector kernel stages the whole of K at once and refuses this width; the batched one walks K in chunks
    for b in range(nb):
        one = backend.zeros(M)
        ctx.matmul_quant_assign(one, m, backend.vector(v[b]))
        assert rel_l2(got[b], one.to_numpy()) < 1e-5


@pytest.mark.parametrize("M,K", [(288, 288), (1031, 1600), (9, 32)])
def test_gemv_batch_q8_0_ragged(backend, ctx, M, K):
    rng = np.random.default_rng(M + K)
    blocks = synth.quantize(synth.FMT_Q8_0, synth.normal_matrix(M + K, M, K))
    v = rng.standard_normal((5, K)).astype(np.float32)
    got = run_batch(backend, ctx, GpuQuantMatrix(backend, synth.FMT_Q8_0, M, K, blocks), v)
    w = O.dequantize(synth.FMT_Q8_0, blocks).reshape(M, K).astype(np.float64)
    for b in range(5):
        assert rel_l2(got[b], w @ v[b].astype(np.float64)) < 1e-5


@pytest.mark.parametrize("fmt", FMTS)
def test_gemv_batch_random_bit_patterns_and_ranges(backend, ctx, fmt):
    """Blocks of random bits; vectors of very different magnitudes in one batch (each is scaled on its own), a zero vector
    among them."""
    M, K = 300, 2048
    rng = np.random.default_rng(77 + fmt)
    blocks = synth.random_blocks(fmt, M, K, rng)
    scales = np.array([1e-30, 1e-6, 1.0, 1e4, 1e30, 0.0, 3.0, 1e-3], dtype=np.float64)
    v = (rng.standard_normal((8, K)) * scales[:, None]).astype(np.float32)
    got = run_batch(backend, ctx, GpuQuantMatrix(backend, fmt, M, K, blocks), v)
    w = O.dequantize(fmt, blocks).reshape(M, K).astype(np.float64)
    for b in range(8):
        if scales[b] == 0.0:
            assert np.all(got[b] == 0)
        else:
            assert rel_l2(got[b], w @ v[b].astype(np.float64)) < 1e-5


def test_gemv_batch_is_deterministic_and_f32_matrices_loop(backend, ctx):
    M, K = 1000, 4096
    rng = np.random.default_rng(4)
    v = rng.standard_normal((8, K)).astype(np.float32)
    m = GpuQuantMatrix(backend, synth.FMT_Q4_K, M, K, synth.quantize(synth.FMT_Q4_K, synth.normal_matrix(5, M, K)))
    a, b = run_batch(backend, ctx, m, v), run_batch(backend, ctx, m, v)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    wf = synth.normal_matrix(6, 64, 512)
    mf = GpuQuantMatrix(backend, synth.FMT_F32, 64, 512, wf)
    got = run_batch(backend, ctx, mf, v[:3, :512].copy())
    for i in range(3):
        assert rel_l2(got[i], wf.reshape(64, 512).astype(np.float64) @ v[i, :512].astype(np.float64)) < 1e-5
