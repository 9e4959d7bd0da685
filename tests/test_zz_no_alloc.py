"""The allocation-free attention entry point (slai_attention_static), called through the C ABI.

It exists for hosts that get their device memory once and may not call the CUDA allocator afterwards; its
scratch is a fixed device array inside the library.  The array is shared by all calls and keeps old contents, so
the test makes calls in a row with different shapes and positions and checks each against slai_attention
(same kernel, allocated scratch) and against the CPU oracle, at the tolerance the attention parity tests use; it
also checks the property the entry point exists for: after the first call on the device, further calls leave the
free device memory unchanged.  This file sorts last on purpose: a run that stops at the first failure has then
already exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from slai_b200 import _lib
from slai_b200.ops import BatchedMultiqueryAttentionParams

pytestmark = pytest.mark.gpu


def _inputs(backend, seq, nh, kvm, hs, pos, kv_dtype, seed):
    rng = np.random.default_rng(seed)
    kvd = nh // kvm * hs
    npdt = np.float16 if kv_dtype == _lib.KV_F16 else np.float32
    k = rng.standard_normal((seq, kvd)).astype(npdt)
    v = rng.standard_normal((seq, kvd)).astype(npdt)
    q = rng.standard_normal(nh * hs).astype(np.float32)
    p = BatchedMultiqueryAttentionParams(seq_len=seq, kv_dim=kvd, kv_mul=kvm, n_heads=nh, head_size=hs, pos=pos)
    return k, v, q, p, backend.vector(k, npdt), backend.vector(v, npdt), backend.vector(q)


def _static(backend, p, dq, dk, dv, kv_dtype, out):
    pc = p.to_c()
    return backend.lib.slai_attention_static(backend.h, C.byref(pc), C.c_void_p(dq.ptr), C.c_void_p(dk.ptr), C.c_void_p(dv.ptr), kv_dtype,
                                             C.c_void_p(out.ptr))


def test_static_attention_matches_allocating_entry_and_oracle(backend):
    # first call: many splits (long context, GQA); second call right after: other shape, short context, so stale
    # partials and tickets of the first call would show up if they were not reset
    for args in ((2048, 64, 8, 128, 1500, _lib.KV_F16, 1), (1024, 12, 1, 64, 7, _lib.KV_F32, 2), (4096, 32, 1, 128, 4095, _lib.KV_F16, 3)):
        seq, nh, kvm, hs, pos, kv_dtype, _ = args
        k, v, q, p, dk, dv, dq = _inputs(backend, *args)
        ref, out = backend.zeros(nh * hs), backend.zeros(nh * hs)
        pc = p.to_c()
        backend.check(backend.lib.slai_attention(backend.h, C.byref(pc), C.c_void_p(dq.ptr), C.c_void_p(dk.ptr), C.c_void_p(dv.ptr), kv_dtype,
                                                 C.c_void_p(ref.ptr)))
        backend.check(_static(backend, p, dq, dk, dv, kv_dtype, out))
        ref, out = ref.to_numpy(), out.to_numpy()
        assert np.isfinite(out).all()
        err = np.linalg.norm(out - ref) / np.linalg.norm(ref)
        assert err < 2e-5, (args, err)
        want, _ = O.attention(q, k.astype(np.float32), v.astype(np.float32), seq_len=seq, kv_dim=nh // kvm * hs, kv_mul=kvm, n_heads=nh,
                              head_size=hs, pos=pos)
        err = np.linalg.norm(out - want) / np.linalg.norm(want)
        assert err < 2e-5, (args, err)


def test_static_attention_requests_no_memory_after_the_first_call(backend):
    args = (2048, 32, 4, 128, 1000, _lib.KV_F16, 5)
    k, v, q, p, dk, dv, dq = _inputs(backend, *args)
    out = backend.zeros(32 * 128)
    backend.check(_static(backend, p, dq, dk, dv, _lib.KV_F16, out))  # set-up call (address look-up, kernel image)
    backend.synchronize()
    free0, _ = backend.mem_info()
    for pos in (1001, 1002, 3, 2047):
        p.pos = pos
        backend.check(_static(backend, p, dq, dk, dv, _lib.KV_F16, out))
    backend.synchronize()
    free1, _ = backend.mem_info()
    assert free1 == free0


def test_static_attention_rejects_oversized_shapes_at_any_position(backend):
    dummy = backend.zeros(16)
    # 1024 query heads x 256 dims over a long context needs far more than the 4 MiB array
    seq, nh, hs = 4096, 1024, 256
    for pos in (seq - 1, 0):  # the limit is that of the cache's last position: also refused at position 0
        p = BatchedMultiqueryAttentionParams(seq_len=seq, kv_dim=nh * hs, kv_mul=1, n_heads=nh, head_size=hs, pos=pos)
        rc = _static(backend, p, dummy, dummy, dummy, _lib.KV_F16, dummy)
        assert rc == _lib.ERR_SHAPE
        msg = backend.lib.slai_last_error_string(backend.h).decode()
        assert "slai_attention_static" in msg and "4194304" in msg
    # 64 heads x 256 dims passes at short contexts only by position; with the cache-sized check it is refused from the start
    p = BatchedMultiqueryAttentionParams(seq_len=4096, kv_dim=64 * 256, kv_mul=1, n_heads=64, head_size=256, pos=0)
    assert _static(backend, p, dummy, dummy, dummy, _lib.KV_F16, dummy) == _lib.ERR_SHAPE
