"""The allocation-free attention backward (``cb_attn_bwd_noalloc``, csrc/no_alloc.h) called
through its exported C symbol must reproduce the regular entry point.

Some users of the kernel library run where device memory was handed out once at start-up (for
example to a KV-cache pool that took the rest of HBM) or where ``cudaMalloc`` is unwelcome
because it stalls the device; they cannot supply the scratch buffers the regular entry point
needs.  The variant keeps its scratch inside the library image.  This file is collected last
so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from coeus_b200.ops import _lib
from coeus_b200.ops import attention as A

pytestmark = pytest.mark.gpu


def _call_noalloc(do, q, k, v, o, lse, out, B, S, nh, dh, causal):
    lib = _lib.lib()
    fn = lib.cb_attn_bwd_noalloc
    fn.restype = ctypes.c_int
    st = _lib.status_buffer(q.device)
    return fn(_lib.ptr(do), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse),
              _lib.ptr(out), B, S, nh, dh, do.stride(0), q.stride(0), k.stride(0), v.stride(0),
              o.stride(0), out.stride(0), ctypes.c_float(1.0 / dh ** 0.5), int(causal),
              _lib.ptr(st), _lib.stream_ptr())


@pytest.mark.parametrize("dh,nh", [(64, 4), (128, 2)])
def test_noalloc_matches_regular_entry_point_twice(dh, nh):
    torch.manual_seed(11)
    B, S = 2, 384
    H = nh * dh
    dev = torch.device("cuda", 0)
    for call in range(2):  # the second call reuses the scratch left behind by the first
        qkv = torch.randn(B * S, 3 * H, device=dev).to(torch.bfloat16)
        q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
        o, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=True)
        do = torch.randn(B * S, H, device=dev).to(torch.bfloat16)
        want = torch.empty(B * S, 3 * H, dtype=torch.bfloat16, device=dev)
        A.attention_bwd(do, q, k, v, o, lse, B, S, nh, dh, causal=True, dqkv=want)
        got = torch.full((B * S, 3 * H), float("nan"), dtype=torch.bfloat16, device=dev)
        rc = _call_noalloc(do, q, k, v, o, lse, got, B, S, nh, dh, True)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert _lib.status_buffer(dev).tolist()[0] == 0
        err = (got.float() - want.float()).abs().max().item()
        # dQ is accumulated with fp32 atomics in both paths, so the two results may differ in
        # the last bf16 bit; the tolerance is the one the kernel tests use.
        assert err < 0.02 * want.float().abs().max().item() + 0.03, (call, err)


def test_noalloc_rejects_oversize_problem():
    lib = _lib.lib()
    lib.cb_noalloc_strerror.restype = ctypes.c_char_p
    dev = torch.device("cuda", 0)
    t = torch.zeros(8, dtype=torch.bfloat16, device=dev)
    f = torch.zeros(8, dtype=torch.float32, device=dev)
    # 64 * 2048 * 16 * 64 floats is far beyond the 4 Mi-float scratch: nothing may be launched
    rc = lib.cb_attn_bwd_noalloc(_lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t),
                                 _lib.ptr(f), _lib.ptr(t), 64, 2048, 16, 64, 1024, 1024, 1024,
                                 1024, 1024, 3072, ctypes.c_float(0.125), 1, _lib.ptr(None),
                                 _lib.stream_ptr())
    assert rc == -100
    assert b"maximum" in lib.cb_noalloc_strerror(rc)
    torch.cuda.synchronize()


def test_noalloc_rejects_unsupported_head_dim_before_touching_anything():
    """dh = 32 passes the size check but no kernel covers it: the call must return a negative
    code with nothing enqueued (output untouched, status word clear)."""
    lib = _lib.lib()
    lib.cb_noalloc_strerror.restype = ctypes.c_char_p
    dev = torch.device("cuda", 0)
    B, S, nh, dh = 1, 128, 2, 32
    H = nh * dh
    t = torch.zeros(B * S, H, dtype=torch.bfloat16, device=dev)
    lse = torch.zeros(B * nh * S, dtype=torch.float32, device=dev)
    out = torch.full((B * S, 3 * H), 7.0, dtype=torch.bfloat16, device=dev)
    rc = _call_noalloc(t, t, t, t, t, lse, out, B, S, nh, dh, True)
    assert rc == -1
    assert b"head dimension" in lib.cb_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
    assert _lib.status_buffer(dev).tolist()[0] == 0
