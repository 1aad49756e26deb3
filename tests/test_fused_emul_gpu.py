"""The fused all-gather->GEMM and GEMM->reduce-scatter kernels on ONE GPU, with the "peers" being
other buffers of the same device: checks the gather ring, the tile ordering and the receive-slot
addressing without NVLink, and the bounded wait of the gather when a peer never reports."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(**kw):
    from coeus_b200.parallel.tp import _CommArgs
    c = _CommArgs()
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def _fused(a, w, out, c, N, K, b_mn=True):
    from coeus_b200.ops import _lib
    st = _lib.status_buffer(a.device)
    rc = _lib.lib().cb_gemm_bf16_fused(
        _lib.ptr(a), _lib.ptr(w), _lib.ptr(out), a.shape[0], N, K, a.stride(0), w.stride(0),
        out.stride(0) if out is not None else N, int(b_mn), _lib.ptr(None),
        256 if N > 128 else 128, ctypes.byref(c), _lib.ptr(st), 0, _lib.stream_ptr())
    assert rc == 0


@pytest.mark.parametrize("tp,rank,K,N", [(4, 1, 512, 384), (8, 7, 2048, 768), (2, 0, 264, 128)])
def test_all_gather_gemm_with_local_peers(tp, rank, K, N):
    from coeus_b200.ops import _lib, gemm as G
    dev = torch.device("cuda")
    torch.manual_seed(0)
    Ts = 256
    T = tp * Ts
    truth = torch.randn(T, K, device=dev).bfloat16()           # what the gathered operand must be
    x = torch.zeros(T, K, device=dev, dtype=torch.bfloat16)     # this rank's gather buffer
    x[rank * Ts:(rank + 1) * Ts] = truth[rank * Ts:(rank + 1) * Ts]
    w = (torch.randn(K, N, device=dev) * 0.05).bfloat16()
    out = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
    flags = torch.zeros((T + 127) // 128, dtype=torch.int32, device=dev)
    pflags = torch.zeros(16, dtype=torch.int64, device=dev)
    for epoch in (1, 2):      # twice: counters keep counting
        x[:rank * Ts] = 0
        x[(rank + 1) * Ts:] = 0
        pflags.fill_(epoch)
        c = _args(comm=1, tp=tp, rank=rank, rows_per_shard=Ts, ag_flags=flags.data_ptr(),
                  ag_epoch=epoch, peer_flags=pflags.data_ptr(), peer_expect=epoch,
                  wait_limit_ns=int(2e9))
        for r in range(tp):
            c.ag_src[r] = x.data_ptr() if r == rank else truth.data_ptr()
        _fused(x, w, out, c, N, K)
        torch.cuda.synchronize()
        _lib.check_status(dev)
        assert torch.equal(x, truth)                            # the gather is bitwise
        ref = G.gemm(truth, w, b_mn=True)
        assert torch.equal(out, ref)                            # same GEMM on the same data


def test_gather_wait_runs_out_when_a_peer_never_reports():
    from coeus_b200.foundation.error import CommError
    from coeus_b200.ops import _lib
    dev = torch.device("cuda")
    tp, Ts, K, N = 2, 128, 256, 128
    T = tp * Ts
    x = torch.zeros(T, K, device=dev, dtype=torch.bfloat16)
    other = torch.zeros(T, K, device=dev, dtype=torch.bfloat16)
    w = torch.zeros(K, N, device=dev, dtype=torch.bfloat16)
    out = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
    flags = torch.zeros(2, dtype=torch.int32, device=dev)
    pflags = torch.zeros(16, dtype=torch.int64, device=dev)     # nothing ever sets pflags[1]
    c = _args(comm=1, tp=tp, rank=0, rows_per_shard=Ts, ag_flags=flags.data_ptr(), ag_epoch=1,
              peer_flags=pflags.data_ptr(), peer_expect=1, wait_limit_ns=int(50e6))
    c.ag_src[0], c.ag_src[1] = x.data_ptr(), other.data_ptr()
    _fused(x, w, out, c, N, K)
    torch.cuda.synchronize()
    with pytest.raises(CommError):
        _lib.check_status(dev)
    _lib.check_status(dev)                                       # cleared, context usable
    assert float(torch.ones(8, device=dev).sum()) == 8.0


def test_gemm_reduce_scatter_with_local_slots():
    from coeus_b200.ops import _lib, gemm as G
    dev = torch.device("cuda")
    torch.manual_seed(1)
    tp, rank, Ts, K, N = 4, 2, 256, 320, 512
    T = tp * Ts
    a = torch.randn(T, K, device=dev).bfloat16()
    w = (torch.randn(K, N, device=dev) * 0.05).bfloat16()
    # "rank s's receive slot for this rank" = region s of one local buffer
    slots = torch.zeros(tp, Ts, N, device=dev, dtype=torch.bfloat16)
    c = _args(comm=2, tp=tp, rank=rank, rows_per_shard=Ts, rs_ld=N, wait_limit_ns=int(2e9))
    for s in range(tp):
        c.rs_dst[s] = slots[s].data_ptr()
    _fused(a, w, None, c, N, K)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    ref = G.gemm(a, w, b_mn=True).view(tp, Ts, N)
    assert torch.equal(slots, ref)
