"""Numerics of every hand-written CUDA kernel against the plain PyTorch fp32 restatement of the
same op (the CPU branch of each function in ``coeus_b200.ops``)."""
import math

import pytest
import torch

from coeus_b200.ops import _lib
from coeus_b200.ops import attention as A
from coeus_b200.ops import elementwise as E
from coeus_b200.ops import gemm as G
from coeus_b200.ops import norm as N

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _status_clean():
    assert _lib.status_buffer(torch.device("cuda", 0)).tolist()[0] == 0


def _bf(x):
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 256, 128), (384, 512, 320), (200, 264, 72), (1024, 2048, 512)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_layouts(a_mn, b_mn, shape, bn):
    M, Nn, K = shape
    torch.manual_seed(1)
    a = _bf(torch.randn((K, M) if a_mn else (M, K), device=DEV))
    b = _bf(torch.randn((K, Nn) if b_mn else (Nn, K), device=DEV))
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    ref = G.gemm(a.cpu(), b.cpu(), a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    err = (out.float().cpu() - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 1e-3
    _status_clean()


def test_gemm_epilogues():
    torch.manual_seed(2)
    M, Nn, K = 512, 768, 256
    x = _bf(torch.randn(M, K, device=DEV))
    w = _bf(torch.randn(K, Nn, device=DEV) * 0.05)
    bias = _bf(torch.randn(Nn, device=DEV))
    r = _bf(torch.randn(M, Nn, device=DEV))
    dy = _bf(torch.randn(M, Nn, device=DEV))
    y = G.linear_fwd(x, w, bias, resid=r)
    ref = G.linear_fwd(x.cpu(), w.cpu(), bias.cpu(), resid=r.cpu(), out_dtype=torch.float32)
    assert (y.float().cpu() - ref).abs().max() < 0.05
    pre = torch.empty(M, Nn, device=DEV, dtype=torch.bfloat16)
    y = G.linear_fwd(x, w, bias, epi="gelu", aux_out=pre)
    pre_ref = torch.empty(M, Nn, dtype=torch.float32)
    ref = G.linear_fwd(x.cpu(), w.cpu(), bias.cpu(), epi="gelu", aux_out=pre_ref,
                       out_dtype=torch.float32)
    assert (y.float().cpu() - ref).abs().max() < 0.03
    assert (pre.float().cpu() - pre_ref).abs().max() < 0.03
    dx = G.linear_dgrad(dy, w)
    assert (dx.float().cpu() - dy.float().cpu() @ w.float().cpu().t()).abs().max() < 0.05
    aux = _bf(torch.randn(M, K, device=DEV))
    dx = G.linear_dgrad(dy, w, epi="dgelu", aux_in=aux)
    ref = (dy.float().cpu() @ w.float().cpu().t()) * G._gelu_grad_ref(aux.float().cpu())
    assert (dx.float().cpu() - ref).abs().max() < 0.05
    gw = torch.zeros(K, Nn, device=DEV)
    G.linear_wgrad(x, dy, gw, ksplit=4)
    G.linear_wgrad(x, dy, gw, ksplit=1)
    ref = 2 * (x.float().cpu().t() @ dy.float().cpu())
    assert (gw.cpu() - ref).abs().max() < 1e-2
    yf = G.linear_fwd(x, w, out_dtype=torch.float32)
    assert (yf.cpu() - x.float().cpu() @ w.float().cpu()).abs().max() < 1e-3
    _status_clean()


@pytest.mark.parametrize("H", [64, 768, 1000, 1024, 1536, 2048, 4096])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(H, rms):
    torch.manual_seed(3)
    T = 517
    x = _bf(torch.randn(T, H, device=DEV) * 2 + 0.5)
    g = _bf(torch.randn(H, device=DEV))
    b = None if rms else _bf(torch.randn(H, device=DEV))
    dy = _bf(torch.randn(T, H, device=DEV))
    dres = _bf(torch.randn(T, H, device=DEV))
    y, mean, rstd = N.norm_fwd(x, g, b, 1e-5, rms)
    yr, meanr, rstdr = N.norm_fwd(x.cpu(), g.cpu(), None if b is None else b.cpu(), 1e-5, rms)
    assert (y.float().cpu() - yr.float()).abs().max() < 0.06
    assert (rstd.cpu() - rstdr).abs().max() < 1e-3
    dg = torch.zeros(H, device=DEV)
    db = None if rms else torch.zeros(H, device=DEV)
    dx = N.norm_bwd(dy, x, g, mean, rstd, dg, db, dres, rms)
    dgr = torch.zeros(H)
    dbr = None if rms else torch.zeros(H)
    dxr = N.norm_bwd(dy.cpu(), x.cpu(), g.cpu(), meanr, rstdr, dgr, dbr, dres.cpu(), rms)
    assert (dx.float().cpu() - dxr.float()).abs().max() < 0.08
    assert (dg.cpu() - dgr).abs().max() < 0.02 * dgr.abs().max() + 0.05
    if not rms:
        assert (db.cpu() - dbr).abs().max() < 0.02 * dbr.abs().max() + 0.05
    _status_clean()


@pytest.mark.parametrize("T,H,rms,with_res", [(40000, 1024, False, True), (40000, 1024, True, False),
                                              (9001, 2048, False, True), (9001, 2048, True, True),
                                              (3, 512, False, False), (700, 4096, False, True)])
def test_norm_many_rows_and_column_sums(T, H, rms, with_res):
    """More rows than one round of the persistent warps (every warp's ring of row buffers wraps
    several times), with and without the residual gradient, and the column sums of the result
    taken in the same pass (the width that the row-pipelined kernel does not cover falls back to
    a separate pass)."""
    torch.manual_seed(5)
    x = _bf(torch.randn(T, H, device=DEV) * 1.5 - 0.25)
    g = _bf(torch.randn(H, device=DEV))
    b = None if rms else _bf(torch.randn(H, device=DEV))
    dy = _bf(torch.randn(T, H, device=DEV))
    dres = _bf(torch.randn(T, H, device=DEV)) if with_res else None
    y, mean, rstd = N.norm_fwd(x, g, b, 1e-5, rms)
    xf = x.float()
    if rms:
        rr = torch.rsqrt((xf * xf).mean(-1) + 1e-5)
        xh = xf * rr[:, None]
        yr = xh * g.float()
    else:
        mu = xf.mean(-1)
        rr = torch.rsqrt(((xf - mu[:, None]) ** 2).mean(-1) + 1e-5)
        xh = (xf - mu[:, None]) * rr[:, None]
        yr = xh * g.float() + b.float()
        assert (mean - mu).abs().max() < 1e-3
    assert (rstd - rr).abs().max() < 1e-3 * float(rr.max())
    assert (y.float() - yr).abs().max() < 0.06
    dg = torch.zeros(H, device=DEV)
    db = None if rms else torch.zeros(H, device=DEV)
    cols = torch.zeros(H, device=DEV)
    dx = N.norm_bwd(dy, x, g, mean, rstd, dg, db, dres, rms, colsum=cols)
    dgv = dy.float() * g.float()
    dxr = rr[:, None] * (dgv - (0 if rms else dgv.mean(-1, keepdim=True))
                         - xh * (dgv * xh).mean(-1, keepdim=True))
    if with_res:
        dxr = dxr + dres.float()
    assert (dx.float() - dxr).abs().max() < 0.08
    dgr = (dy.float() * xh).sum(0)
    assert (dg - dgr).abs().max() < 0.02 * float(dgr.abs().max()) + 0.05
    if not rms:
        dbr = dy.float().sum(0)
        assert (db - dbr).abs().max() < 0.02 * float(dbr.abs().max()) + 0.05
    cr = dxr.sum(0)
    assert (cols - cr).abs().max() < 4e-3 * float(cr.abs().max()) + 0.1
    dx2 = N.norm_bwd(dy, x, g, mean, rstd, torch.zeros_like(dg), None if rms else torch.zeros_like(db),
                     dres, rms)
    assert torch.equal(dx, dx2)
    _status_clean()


def test_embedding_and_positions():
    torch.manual_seed(4)
    V, H, S, B = 1000, 256, 64, 3
    table = _bf(torch.randn(V, H, device=DEV))
    ids = torch.randint(0, V, (B * S,), device=DEV)
    pe = E.sinusoid_table(S, H, DEV)
    per = E.sinusoid_table(S, H, "cpu")
    assert (pe.cpu() - per).abs().max() < 2e-4
    out = E.embed_fwd(ids, table, pe, S)
    ref = E.embed_fwd(ids.cpu(), table.cpu(), per, S)
    assert (out.float().cpu() - ref.float()).abs().max() < 0.03
    dy = _bf(torch.randn(B * S, H, device=DEV))
    gt = torch.zeros(V, H, device=DEV)
    E.embed_bwd(ids, dy, gt)
    gtr = torch.zeros(V, H)
    E.embed_bwd(ids.cpu(), dy.cpu(), gtr)
    assert (gt.cpu() - gtr).abs().max() < 1e-4
    _status_clean()


def test_embedding_out_of_range_sets_status():
    V, H = 100, 64
    table = _bf(torch.randn(V, H, device=DEV))
    ids = torch.tensor([1, 2, 100], device=DEV)
    out = E.embed_fwd(ids, table, None, 3)
    torch.cuda.synchronize()
    st = _lib.status_buffer(torch.device("cuda", 0))
    assert st.tolist()[:2] == [2, 2]
    assert out[2].abs().max() == 0
    st.zero_()


@pytest.mark.parametrize("V", [512, 32000])
def test_cross_entropy(V):
    torch.manual_seed(5)
    T = 300
    logits = _bf(torch.randn(T, V, device=DEV) * 3)
    tgt = torch.randint(0, V, (T,), device=DEV)
    tgt[5] = -100
    lc, tc = logits.clone().cpu(), tgt.cpu()
    loss = E.cross_entropy_fwd_bwd(logits, tgt, 1.0 / T)
    lr = E.cross_entropy_fwd_bwd(lc, tc, 1.0 / T)
    assert (loss.cpu() - lr).abs().max() < 2e-3
    assert (logits.float().cpu() - lc.float()).abs().max() < 2e-4
    # vocab-parallel halves on two shards reproduce the fused result
    full = _bf(torch.randn(T, V, device=DEV) * 3)
    half = V // 2
    stats = [E.cross_entropy_stats(full[:, i * half:(i + 1) * half], tgt, i * half) for i in range(2)]
    m = torch.maximum(stats[0][:, 0], stats[1][:, 0])
    s = sum(st[:, 1] * torch.exp(st[:, 0] - m) for st in stats)
    lse = m + torch.log(s)
    tl = stats[0][:, 2] + stats[1][:, 2]
    ref = torch.nn.functional.cross_entropy(full.float(), tgt, reduction="none", ignore_index=-100)
    assert ((lse - tl) * (tgt >= 0) - ref).abs().max() < 2e-3


def test_adamw_matches_torch():
    torch.manual_seed(6)
    n = 100003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    pb = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in (1, 2, 3):
        ref.grad = g.clone()
        opt.step()
        E.adamw_step(p, m, v, g, pb, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                     step=step)
    assert (p - ref.data).abs().max() < 1e-5
    assert (pb.float() - p).abs().max() < 0.02


def test_activations_softmax_rope_colsum_init():
    torch.manual_seed(7)
    x = _bf(torch.randn(333, 512, device=DEV) * 2)
    dy = _bf(torch.randn(333, 512, device=DEV))
    assert (E.gelu_fwd(x).float().cpu() - E.gelu_fwd(x.cpu()).float()).abs().max() < 0.02
    assert (E.gelu_bwd(x, dy).float().cpu() - E.gelu_bwd(x.cpu(), dy.cpu()).float()).abs().max() < 0.03
    # the same with the column sums of the result (a bias gradient) added in the same pass
    acc = torch.full((512,), 0.5, device=DEV)
    dxf = E.gelu_bwd(x, dy, acc)
    assert torch.equal(dxf, E.gelu_bwd(x, dy))
    assert (acc.cpu() - 0.5 - dxf.float().cpu().sum(0)).abs().max() < 1e-2
    gu = _bf(torch.randn(100, 1024, device=DEV))
    d2 = _bf(torch.randn(100, 512, device=DEV))
    assert (E.swiglu_fwd(gu).float().cpu() - E.swiglu_fwd(gu.cpu()).float()).abs().max() < 0.03
    assert (E.swiglu_bwd(gu, d2).float().cpu() - E.swiglu_bwd(gu.cpu(), d2.cpu()).float()).abs().max() < 0.05
    z = torch.randn(77, 1000, device=DEV)
    assert (E.softmax_rows(z).cpu() - torch.softmax(z.cpu(), -1)).abs().max() < 1e-6
    q = _bf(torch.randn(64, 4 * 64, device=DEV))
    qc = q.clone().cpu()
    E.rope_(q, 4, 64, 16, pos_offset=3)
    E.rope_(qc, 4, 64, 16, pos_offset=3)
    assert (q.float().cpu() - qc.float()).abs().max() < 0.03
    cs = torch.zeros(512, device=DEV)
    E.colsum_into(x, cs)
    assert (cs.cpu() - x.float().cpu().sum(0)).abs().max() < 1e-2
    p = torch.empty(5000, device=DEV)
    E.sin_init_(p, 768, index_offset=20_000_000)
    pr = torch.empty(5000)
    E.sin_init_(pr, 768, index_offset=20_000_000)
    assert (p.cpu() - pr).abs().max() < 1e-5


@pytest.mark.parametrize("dh", [64, 128])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("S", [128, 200, 512])
def test_attention_fwd_bwd(dh, causal, S):
    torch.manual_seed(8)
    B, nh = 2, 3
    H = nh * dh
    qkv = _bf(torch.randn(B * S, 3 * H, device=DEV))
    q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
    o, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=causal)
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    orf, lser = A.attention_fwd(qc, kc, vc, B, S, nh, dh, causal=causal)
    torch.cuda.synchronize()
    _status_clean()
    assert (o.float().cpu() - orf.float()).abs().max() < 0.03
    assert (lse.cpu() - lser).abs().max() < 0.02
    do = _bf(torch.randn(B * S, H, device=DEV))
    dq, dk, dv = A.attention_bwd(do, q, k, v, o, lse, B, S, nh, dh, causal=causal)
    dqr, dkr, dvr = A.attention_bwd(do.cpu(), qc, kc, vc, orf, lser, B, S, nh, dh, causal=causal)
    torch.cuda.synchronize()
    _status_clean()
    for got, ref, name in ((dq, dqr, "dq"), (dk, dkr, "dk"), (dv, dvr, "dv")):
        err = (got.float().cpu() - ref.float()).abs().max().item()
        assert err < 0.02 * ref.float().abs().max().item() + 0.03, (name, err)


@pytest.mark.parametrize("dh,B,nh,S,causal", [
    (64, 1, 2, 1152, True), (64, 1, 2, 1100, True), (64, 1, 2, 640, False), (128, 1, 2, 1152, True),
    (64, 4, 16, 512, True),      # 256 work items: persistent CTAs chain several, K/V buffers alternate
    (64, 8, 16, 300, True),      # 384 items of one to three steps, ragged last tile
    (64, 3, 20, 256, False),     # 120 + items of equal length
    (64, 5, 32, 128, True),      # 160 single-step items
])
def test_attention_bwd_many_query_tiles(dh, B, nh, S, causal):
    """Many query tiles per K/V tile (every ring -- query stages, dS^T and dQ buffers -- wraps
    around several times, with a ragged last tile in one case) and more work items than CTAs."""
    torch.manual_seed(18)
    H = nh * dh
    qkv = _bf(torch.randn(B * S, 3 * H, device=DEV))
    q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
    o, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=causal)
    do = _bf(torch.randn(B * S, H, device=DEV))
    dq, dk, dv = A.attention_bwd(do, q, k, v, o, lse, B, S, nh, dh, causal=causal)
    dqr, dkr, dvr = A.attention_bwd(do.cpu(), q.cpu(), k.cpu(), v.cpu(), o.cpu(), lse.cpu(), B, S,
                                    nh, dh, causal=causal)
    torch.cuda.synchronize()
    _status_clean()
    for got, ref, name in ((dq, dqr, "dq"), (dk, dkr, "dk"), (dv, dvr, "dv")):
        err = (got.float().cpu() - ref.float()).abs().max().item()
        assert err < 0.02 * ref.float().abs().max().item() + 0.03, (name, err)


@pytest.mark.parametrize("dh,nh,nkv,B,S,causal", [
    (64, 4, 4, 1, 384, True),       # three query tiles: the last pair has one tile only
    (64, 16, 16, 4, 1024, True),    # 256 work items: persistent CTAs take several each
    (64, 8, 2, 2, 1000, True),      # grouped-query attention, ragged last tile
    (128, 4, 1, 2, 640, True),      # multi-query, dh 128, five query tiles
    (128, 2, 2, 3, 512, False),
    (64, 3, 3, 2, 77, False),
    # odd numbers of query tiles with more work items than CTAs: a CTA's first item has a single
    # query tile, so one softmax warpgroup sits that item out and joins at the next
    (64, 16, 16, 8, 300, True),
    (64, 16, 16, 8, 384, False),
    (64, 16, 4, 8, 640, True),
    (128, 8, 8, 8, 640, True),
    (128, 8, 8, 6, 384, False),
])
def test_attention_fwd_shapes_and_grouped_query(dh, nh, nkv, B, S, causal):
    torch.manual_seed(9)
    H, Hkv = nh * dh, nkv * dh
    qkv = _bf(torch.randn(B * S, H + 2 * Hkv, device=DEV))
    q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
    orf, lser = A.attention_fwd(q.cpu(), k.cpu(), v.cpu(), B, S, nh, dh, causal=causal)
    before = A.FWD_POLY
    try:
        for poly in (0, 1):
            A.FWD_POLY = poly
            o, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=causal)
            torch.cuda.synchronize()
            _status_clean()
            assert (o.float().cpu() - orf.float()).abs().max() < 0.03, poly
            assert (lse.cpu() - lser).abs().max() < 0.02, poly
    finally:
        A.FWD_POLY = before


@pytest.mark.parametrize("dh,nh,nkv,B,S,causal", [
    (64, 4, 4, 2, 256, True), (64, 6, 2, 1, 384, True), (64, 3, 3, 2, 200, False),
    (128, 2, 2, 2, 256, True), (128, 4, 1, 1, 320, False), (64, 16, 16, 8, 256, True),
])
def test_attention_dropout_inside_the_flash_kernels(dh, nh, nkv, B, S, causal):
    """Dropout on the probabilities applied by the forward and backward flash kernels themselves
    (mask recomputed from the element index, nothing stored) against the materialised fp32
    restatement with the same mask."""
    torch.manual_seed(21)
    H, Hkv = nh * dh, nkv * dh
    thr, key = E.dropout_threshold(0.2), E.dropout_key(7, 3, 1, 0, 5, 2)
    qkv = _bf(torch.randn(B * S, H + 2 * Hkv, device=DEV))
    q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
    assert A.flash_dropout_ok(q, S, dh)
    o, lse = A.attention_fwd(q, k, v, B, S, nh, dh, causal=causal, dropout=(thr, key))
    orf, lser = A.attention_dropout_fwd(q.cpu(), k.cpu(), v.cpu(), B, S, nh, dh, thr, key,
                                        causal=causal)
    torch.cuda.synchronize()
    _status_clean()
    assert (o.float().cpu() - orf.float()).abs().max() < 0.04
    assert (lse.cpu() - lser).abs().max() < 0.02
    # a fifth of the probabilities is gone: the output differs from the one without dropout
    o0, _ = A.attention_fwd(q, k, v, B, S, nh, dh, causal=causal)
    assert (o.float() - o0.float()).abs().max() > 0.05
    if nkv != nh:
        return               # the backward kernels take expanded K/V heads (the model sums them)
    do = _bf(torch.randn(B * S, H, device=DEV))
    got = A.attention_bwd(do, q, k, v, o, lse, B, S, nh, dh, causal=causal, dropout=(thr, key))
    ref = A.attention_dropout_bwd(do.cpu(), q.cpu(), k.cpu(), v.cpu(), orf, lser, B, S, nh, dh,
                                  thr, key, causal=causal)
    torch.cuda.synchronize()
    _status_clean()
    for g_, r_, name in zip(got, ref, ("dq", "dk", "dv")):
        err = (g_.float().cpu() - r_.float()).abs().max().item()
        assert err < 0.02 * r_.float().abs().max().item() + 0.04, (name, err)


def test_dropout_mask_is_the_same_on_the_device_in_the_gemm_and_on_the_host():
    """One mask function in three places: the stand-alone kernel, the GEMM epilogue (dropout on
    the value before the residual is added) and the tensor-op restatement on the host."""
    torch.manual_seed(3)
    thr, key = E.dropout_threshold(0.3), E.dropout_key(11, 5, 1, 0, 2, 1)
    x = _bf(torch.randn(300, 256, device=DEV))
    got = E.dropout_apply(x, thr, key)
    want = E.dropout_apply(x.cpu(), thr, key)
    torch.cuda.synchronize()
    _status_clean()
    assert torch.equal(got.cpu(), want)
    kept = float((got != 0).float().mean())
    assert abs(kept - (1 - thr / 256)) < 0.02
    a = _bf(torch.randn(384, 128, device=DEV))
    w = _bf(torch.randn(128, 256, device=DEV) * 0.1)
    bias = _bf(torch.randn(256, device=DEV))
    resid = _bf(torch.randn(384, 256, device=DEV))
    y = G.linear_fwd(a, w, bias, resid=resid, dropout=(thr, key))
    yr = G.linear_fwd(a.cpu(), w.cpu(), bias.cpu(), resid=resid.cpu(), dropout=(thr, key))
    torch.cuda.synchronize()
    _status_clean()
    assert (y.float().cpu() - yr.float()).abs().max() < 0.06
    # where the mask dropped the value only the residual is left, exactly
    keep = E.dropout_mask(384, 256, thr, key)
    assert torch.equal(y.cpu()[~keep], resid.cpu()[~keep])


def test_normal_init_matches_cpu_generator():
    from coeus_b200.ops import elementwise as E
    n = 1_000_003
    ref = E.normal_init_(torch.empty(n), seed=(7 << 32) | 99, std=0.02)
    got = E.normal_init_(torch.empty(n, device="cuda"), seed=(7 << 32) | 99, std=0.02)
    torch.cuda.synchronize()
    assert (got.cpu() - ref).abs().max() < 2e-6
    part = E.normal_init_(torch.empty(4097, device="cuda"), seed=(7 << 32) | 99, std=0.02,
                          index_offset=333_333)
    assert torch.equal(part, got[333_333:333_333 + 4097])


@pytest.mark.parametrize("Gn,M,N,K", [(3, 128, 192, 64), (4, 256, 512, 128), (2, 384, 264, 192)])
def test_grouped_gemm_matches_per_group_reference(Gn, M, N, K):
    """All three products of a stacked linear layer (forward, data gradient, weight gradient) in
    one launch each, against fp32 matmuls per group; M = 256 also exercises CTA pairs."""
    torch.manual_seed(Gn * 1000 + M)
    x = torch.randn(Gn, M, K, device="cuda").bfloat16()
    w = (torch.randn(Gn, K, N, device="cuda") / math.sqrt(K)).bfloat16()     # [in, out] per group
    dy = torch.randn(Gn, M, N, device="cuda").bfloat16()
    y = G.gemm_grouped(x, w, b_mn=True)
    ref = torch.bmm(x.float(), w.float())
    assert (y.float() - ref).abs().max() <= 0.02 * ref.abs().max()
    if N % 64 == 0:
        dx = G.gemm_grouped(dy, w, b_mn=False)
        ref = torch.bmm(dy.float(), w.float().transpose(1, 2))
        assert (dx.float() - ref).abs().max() <= 0.02 * ref.abs().max()
    # the weight gradient's output rows are the input features: one launch when K is a multiple
    # of 128, one per group otherwise
    gw = torch.zeros(Gn, K, N, device="cuda")
    G.linear_wgrad_grouped(x, dy, gw)
    G.linear_wgrad_grouped(x, dy, gw)
    ref = 2 * torch.bmm(x.float().transpose(1, 2), dy.float())
    assert (gw - ref).abs().max() <= 0.01 * ref.abs().max()
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))


def test_kernels_without_atomics_are_bitwise_repeatable():
    """A cheap race detector: kernels whose reduction order is fixed must give the same bits on
    every run (GEMM without split-K, grouped GEMM, attention forward, norm forward, cross-entropy,
    AdamW)."""
    torch.manual_seed(3)
    x = torch.randn(1000, 512, device="cuda").bfloat16()
    w = torch.randn(512, 768, device="cuda").bfloat16()
    xg = torch.randn(4, 256, 128, device="cuda").bfloat16()
    wg = torch.randn(4, 128, 320, device="cuda").bfloat16()
    qkv = torch.randn(2 * 300, 3 * 256, device="cuda").bfloat16()
    scale = torch.randn(512, device="cuda").bfloat16()
    logits = torch.randn(333, 1000, device="cuda").bfloat16()
    tgt = torch.randint(0, 1000, (333,), device="cuda")

    def run():
        y = G.linear_fwd(x, w, epi="gelu")
        yg = G.gemm_grouped(xg, wg, b_mn=True)
        o, lse = A.attention_fwd(qkv[:, :256], qkv[:, 256:512], qkv[:, 512:], 2, 300, 4, 64)
        n, mean, rstd = N.norm_fwd(x, scale, None, 1e-5, True)
        lg = logits.clone()
        loss = E.cross_entropy_fwd_bwd(lg, tgt, 1.0 / 333, vocab=1000)
        return [y, yg, o, lse, n, rstd, lg, loss]

    first = run()
    for _ in range(5):
        for a, b in zip(first, run()):
            assert torch.equal(a, b)
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda", 0))
