"""Failure reporting, several contexts in one process, recorded passes and the single-GPU stand-in for the
tensor-parallel exchange.  Nothing here faults or hangs a GPU: the time-out test polls a tag that nothing writes,
with a short limit, and the kernel returns on its own."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import synth, _lib
from slai_b200._lib import SlaiError
from slai_b200.ops import Backend, BatchedMultiqueryAttentionParams, GpuQuantMatrix, LlmContext
from helpers import rel_l2

pytestmark = pytest.mark.gpu


def _exchange_inputs(backend, fmt, M, K, seed):
    """Row-parallel W (M x K) cut into two K halves, a residual, and a consumer matrix W2 (M2 x M)."""
    rng = np.random.default_rng(seed)
    w = synth.normal_matrix(seed, M, K)
    halves = [np.ascontiguousarray(w[:, :K // 2]), np.ascontiguousarray(w[:, K // 2:])]
    blocks = [synth.quantize(fmt, h) for h in halves]
    v = rng.standard_normal(K).astype(np.float32)
    x = rng.standard_normal(M).astype(np.float32)
    M2 = 48
    b2 = synth.quantize(fmt, synth.normal_matrix(seed + 1, M2, M))
    nw = (1.0 + 0.1 * rng.standard_normal(M)).astype(np.float32)
    return blocks, v, x, b2, nw, M2


@pytest.mark.parametrize("fmt", [synth.FMT_Q4_K, synth.FMT_Q8_0])
def test_loopback_exchange_matches_oracle(fmt):
    """Two ranks played one after the other on one GPU: partial products stored into the exchange region, summed in
    rank order by the consuming kernel while it stages its input."""
    backend = Backend(0)
    ctx = LlmContext(backend)
    M, K = 512, 1024
    blocks, v, x, b2, nw, M2 = _exchange_inputs(backend, fmt, M, K, 11)
    mats = [GpuQuantMatrix(backend, fmt, M, K // 2, b) for b in blocks]
    m2 = GpuQuantMatrix(backend, fmt, M2, M, b2)
    dv = [backend.vector(v[:K // 2]), backend.vector(v[K // 2:])]
    dx, dnw = backend.vector(x), backend.vector(nw)
    out, s = backend.zeros(M2), backend.zeros(M)
    for token in range(2):  # two tokens: the tags of the second must not be satisfied by the first token's data
        for idx in range(2):
            ctx.peer_loopback(2, 0)
            if idx == 0:
                ctx.token_tick()
            ctx.matmul_quant_partial(mats[0], dv[0], dx, idx, 2)
            ctx.peer_loopback(2, 1)
            ctx.matmul_quant_partial(mats[1], dv[1], None, idx, 2)
            ctx.matmul_quant_reduced(out, m2, dnw, 1e-5, idx, 2, s)
            backend.synchronize()
            want_s = x.astype(np.float64)
            for b, vv in zip(blocks, (v[:K // 2], v[K // 2:])):
                want_s = want_s + O.dequantize(fmt, b).reshape(M, K // 2).astype(np.float64) @ vv.astype(np.float64)
            assert rel_l2(s.to_numpy(), want_s) < 1e-5
            xb = O.rms_norm(want_s.astype(np.float32), nw, 1e-5)
            want = O.dequantize(fmt, b2).reshape(M2, M).astype(np.float64) @ xb.astype(np.float64)
            assert rel_l2(out.to_numpy(), want) < 1e-3
    backend.close()


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """A consumer whose second rank never stores its partial: the poll gives up after the (shortened) limit, the
    kernel returns, the next synchronisation reports SLAI_ERR_TIMEOUT once, and the context works afterwards."""
    backend = Backend(0)
    ctx = LlmContext(backend)
    fmt, M, K = synth.FMT_Q4_K, 256, 512
    blocks, v, x, b2, nw, M2 = _exchange_inputs(backend, fmt, M, K, 5)
    m0 = GpuQuantMatrix(backend, fmt, M, K // 2, blocks[0])
    m2 = GpuQuantMatrix(backend, fmt, M2, M, b2)
    dv0, dx, dnw = backend.vector(v[:K // 2]), backend.vector(x), backend.vector(nw)
    out, s = backend.zeros(M2), backend.zeros(M)
    with pytest.raises(SlaiError):
        backend.set_wait_limit(3)  # refused: shorter than a healthy launch needs
    backend.set_wait_limit(2000)
    ctx.peer_loopback(2, 0)
    ctx.token_tick()
    ctx.matmul_quant_partial(m0, dv0, dx, 0, 2)
    ctx.matmul_quant_reduced(out, m2, dnw, 1e-5, 0, 2, s)  # rank 1 never arrives
    with pytest.raises(SlaiError) as e:
        backend.synchronize()
    assert e.value.code == _lib.ERR_TIMEOUT and "tensor-parallel peer" in str(e.value)
    backend.synchronize()  # the flag was cleared: reported once
    backend.set_wait_limit(1 << 20)
    y = backend.zeros(M2)
    xv = backend.vector(np.ones(M, np.float32))
    ctx.matmul_quant_assign(y, m2, xv)
    backend.synchronize()
    want = O.dequantize(fmt, b2).reshape(M2, M).astype(np.float64).sum(axis=1)
    assert rel_l2(y.to_numpy(), want) < 1e-3
    backend.close()


def test_two_contexts_on_two_gpus_in_one_process():
    """Kernel attributes are per device and every entry point selects its context's device: a second context on
    another GPU runs the large-shared-memory GEMV and attention, interleaved with the first, from one thread."""
    lib = _lib.load()
    if lib.slai_device_count() < 2:
        pytest.skip("needs two GPUs")
    bs = [Backend(0), Backend(1)]
    fmt, M, K = synth.FMT_Q4_K, 320, 4096
    blocks = synth.quantize(fmt, synth.normal_matrix(3, M, K))
    v = np.random.default_rng(3).standard_normal(K).astype(np.float32)
    want = O.dequantize(fmt, blocks).reshape(M, K).astype(np.float64) @ v.astype(np.float64)
    mats = [GpuQuantMatrix(b, fmt, M, K, blocks) for b in bs]
    outs = [b.zeros(M) for b in bs]
    vs = [b.vector(v) for b in bs]
    for rnd in range(2):
        for i in (0, 1, 1, 0):
            LlmContext(bs[i]).matmul_quant_assign(outs[i], mats[i], vs[i])
    seq, nh, hs, pos = 256, 8, 64, 200
    rng = np.random.default_rng(9)
    kc = rng.standard_normal((seq, nh * hs)).astype(np.float32)
    vc = rng.standard_normal((seq, nh * hs)).astype(np.float32)
    q = rng.standard_normal(nh * hs).astype(np.float32)
    p = BatchedMultiqueryAttentionParams(seq_len=seq, kv_dim=nh * hs, kv_mul=1, n_heads=nh, head_size=hs, pos=pos)
    xbs = []
    for b in bs:
        xb = b.zeros(nh * hs)
        LlmContext(b).attention(p, b.vector(q), b.vector(kc), b.vector(vc), xb)
        xbs.append(xb)
    want_att, _ = O.attention(q, kc, vc, seq_len=seq, kv_dim=nh * hs, kv_mul=1, n_heads=nh, head_size=hs, pos=pos)
    for i, b in enumerate(bs):
        b.synchronize()
        assert rel_l2(outs[i].to_numpy(), want) < 1e-3
        assert rel_l2(xbs[i].to_numpy(), want_att) < 2e-5
    for b in bs:
        b.close()


def test_recorded_pass_with_attention_replays(backend, ctx):
    """slai_kv_append + slai_attention recorded once and replayed: the position travels by value and the scratch the
    recorded kernels point at stays allocated even when a later eager call needs a larger one."""
    seq, nh, kvm, hs, pos = 512, 8, 2, 64, 300
    kvd = nh // kvm * hs
    rng = np.random.default_rng(4)
    kc_h = rng.standard_normal((seq, kvd)).astype(np.float32)
    vc_h = rng.standard_normal((seq, kvd)).astype(np.float32)
    k_new, v_new = rng.standard_normal(kvd).astype(np.float32), rng.standard_normal(kvd).astype(np.float32)
    q = rng.standard_normal(nh * hs).astype(np.float32)
    kc, vc = backend.vector(kc_h), backend.vector(vc_h)
    dk, dv, dq = backend.vector(k_new), backend.vector(v_new), backend.vector(q)
    p = BatchedMultiqueryAttentionParams(seq_len=seq, kv_dim=kvd, kv_mul=kvm, n_heads=nh, head_size=hs, pos=pos)
    eager = backend.zeros(nh * hs)
    ctx.kv_append(kc, vc, dk, dv, kvd, pos)
    ctx.attention(p, dq, kc, vc, eager)
    backend.synchronize()
    want = eager.to_numpy()
    out = backend.zeros(nh * hs)
    with backend.record() as rec:
        ctx.kv_append(kc, vc, dk, dv, kvd, pos)
        ctx.attention(p, dq, kc, vc, out)
    # an eager call that needs more scratch than anything before it: the recorded pass must not lose its buffer
    big = BatchedMultiqueryAttentionParams(seq_len=4096, kv_dim=32 * 128, kv_mul=1, n_heads=32, head_size=128, pos=4000)
    bk = backend.zeros(4096 * 32 * 128)
    ctx.attention(big, backend.zeros(32 * 128), bk, bk, backend.zeros(32 * 128))
    backend.synchronize()
    for _ in range(2):
        backend.check(backend.lib.slai_memset(backend.h, C.c_void_p(out.ptr), 0, out.nbytes))
        rec.launch(1)
        backend.synchronize()
        assert np.array_equal(out.to_numpy(), want)
    kc_h[pos], vc_h[pos] = k_new, v_new
    ref, _ = O.attention(q, kc_h, vc_h, seq_len=seq, kv_dim=kvd, kv_mul=kvm, n_heads=nh, head_size=hs, pos=pos)
    assert rel_l2(want, ref) < 2e-5
    rec.close()
