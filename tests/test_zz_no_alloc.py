"""The allocation-free attention entry point (slai_attention_static), called through the C ABI.

It exists for hosts that get their device memory once and may not call the CUDA allocator afterwards; its
scratch is a fixed device array inside the library.  The array is shared by all calls and keeps old contents, so
the test makes two calls in a row with different shapes and positions and checks each against slai_attention
(same kernel, allocated scratch), at the tolerance the attention parity tests use.  This file sorts last on
purpose: a run that stops at the first failure has then already exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

from slai_b200 import _lib
from slai_b200.ops import BatchedMultiqueryAttentionParams, LlmContext

pytestmark = pytest.mark.gpu


def _both(backend, seq, nh, kvm, hs, pos, kv_dtype, seed):
    rng = np.random.default_rng(seed)
    kvd = nh // kvm * hs
    npdt = np.float16 if kv_dtype == _lib.KV_F16 else np.float32
    kc = backend.vector(rng.standard_normal((seq, kvd)).astype(npdt), npdt)
    vc = backend.vector(rng.standard_normal((seq, kvd)).astype(npdt), npdt)
    q = backend.vector(rng.standard_normal(nh * hs).astype(np.float32))
    p = BatchedMultiqueryAttentionParams(seq_len=seq, kv_dim=kvd, kv_mul=kvm, n_heads=nh, head_size=hs, pos=pos).to_c()
    ref, out = backend.zeros(nh * hs), backend.zeros(nh * hs)
    lib = backend.lib
    backend.check(lib.slai_attention(backend.h, C.byref(p), C.c_void_p(q.ptr), C.c_void_p(kc.ptr), C.c_void_p(vc.ptr), kv_dtype,
                                     C.c_void_p(ref.ptr)))
    backend.check(lib.slai_attention_static(backend.h, C.byref(p), C.c_void_p(q.ptr), C.c_void_p(kc.ptr), C.c_void_p(vc.ptr),
                                            kv_dtype, C.c_void_p(out.ptr)))
    return ref.to_numpy(), out.to_numpy()


def test_static_attention_matches_allocating_entry_twice(backend):
    # first call: many splits (long context, GQA); second call right after: other shape, short context, so stale
    # partials and tickets of the first call would show up if they were not reset
    for args in ((2048, 64, 8, 128, 1500, _lib.KV_F16, 1), (1024, 12, 1, 64, 7, _lib.KV_F32, 2), (4096, 32, 1, 128, 4095, _lib.KV_F16, 3)):
        ref, out = _both(backend, *args)
        assert np.isfinite(out).all()
        err = np.linalg.norm(out - ref) / np.linalg.norm(ref)
        assert err < 2e-5, (args, err)


def test_static_attention_rejects_oversized_shapes(backend):
    # 1024 query heads x 256 dims over a long context needs far more than the 4 MiB array
    seq, nh, hs = 4096, 1024, 256
    p = BatchedMultiqueryAttentionParams(seq_len=seq, kv_dim=nh * hs, kv_mul=1, n_heads=nh, head_size=hs, pos=seq - 1).to_c()
    dummy = backend.zeros(16)
    rc = backend.lib.slai_attention_static(backend.h, C.byref(p), C.c_void_p(dummy.ptr), C.c_void_p(dummy.ptr), C.c_void_p(dummy.ptr),
                                           _lib.KV_F16, C.c_void_p(dummy.ptr))
    assert rc == _lib.ERR_SHAPE
    msg = backend.lib.slai_last_error_string(backend.h).decode()
    assert "slai_attention_static" in msg and "4194304" in msg
