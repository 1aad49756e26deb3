"""Times one kernel on one shape with CUDA events and reports it against the roofline.

    python -m coeus_b200.utils.kernel_bench gemm --m 16384 --n 4096 --k 1024 --layout fwd
    python -m coeus_b200.utils.kernel_bench attn_fwd --batch 8 --heads 16 --seq 2048 --dh 64
    python -m coeus_b200.utils.kernel_bench norm_bwd --tokens 16384 --hidden 1024

Warm-up iterations first, then timed iterations bracketed by synchronisations; inputs are larger
than the L2 cache or, for small ones, ``--flush-l2`` writes a 256 MB buffer between iterations.
The denominators are the measured copy bandwidth and cuBLAS bf16 throughput of the machine when
``MEASURED_PEAKS.json`` is present next to the package, else the stated fallback.  This is also
the program the committed ``ncu`` summaries under ``profiles/`` were captured from (with small
``--iters``)."""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, warmup: int, iters: int, flush: bool):
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if scratch is not None:
            scratch.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attn_fwd", "attn_bwd", "norm_fwd", "norm_bwd",
                                       "cross_entropy", "adamw", "decode_attn", "rope", "softmax",
                                       "swiglu", "gelu", "embed", "rmsnorm_fwd", "rmsnorm_bwd",
                                       "moe_route", "allreduce_local", "kv_write", "argmax",
                                       "normal_init", "colsum", "moe_gather", "moe_combine"])
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--layout", default="fwd", choices=["fwd", "dgrad", "wgrad"])
    ap.add_argument("--epi", default="none", choices=["none", "gelu", "bias"])
    ap.add_argument("--ksplit", type=int, default=0)
    ap.add_argument("--groups", type=int, default=1,
                    help="gemm: number of stacked groups (experts); m, n, k are per group and "
                         "--compare-torch then times one launch per group instead")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--dh", type=int, default=64)
    ap.add_argument("--attn-poly", type=int, default=None,
                    help="0: every exponential on the special-function unit; 1: a share as polynomial")
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--numel", type=int, default=64 << 20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--compare-torch", action="store_true")
    ap.add_argument("--variant", type=int, default=-1, help="kernel variant (norm_bwd: 0, 1, 2 rows in registers, 3 row-pipelined; norm_fwd: 0, 1)")
    a = ap.parse_args(argv)
    from ..ops import attention as A
    from ..ops import decode as D
    from ..ops import elementwise as E
    from ..ops import gemm as G
    from ..ops import norm as N
    dev = "cuda"
    bf = torch.bfloat16
    if a.variant >= 0 and a.kernel in ("norm_bwd", "rmsnorm_bwd"):
        from ..ops import _lib
        _lib.lib().cb_norm_bwd_variant(a.variant)
    if a.variant >= 0 and a.kernel in ("norm_fwd", "rmsnorm_fwd"):
        from ..ops import _lib
        _lib.lib().cb_norm_fwd_variant(a.variant)
    hbm, tf, src = peaks()
    flops = nbytes = 0.0
    torch_fn = None
    if a.kernel == "gemm" and a.groups > 1:
        Gn, M, Nn, K = a.groups, a.m, a.n, a.k
        w = torch.randn(Gn, K, Nn, device=dev).to(bf)
        if a.layout == "fwd":
            x = torch.randn(Gn, M, K, device=dev).to(bf)
            obuf = torch.empty(Gn, M, Nn, device=dev, dtype=bf)
            fn = lambda: G.gemm_grouped(x, w, b_mn=True, out=obuf)  # noqa: E731
            torch_fn = lambda: [G.gemm(x[g], w[g], b_mn=True, out=obuf[g]) for g in range(Gn)]  # noqa: E731
        elif a.layout == "dgrad":
            dy = torch.randn(Gn, M, Nn, device=dev).to(bf)
            obuf = torch.empty(Gn, M, K, device=dev, dtype=bf)
            fn = lambda: G.gemm_grouped(dy, w, out=obuf)  # noqa: E731
            torch_fn = lambda: [G.gemm(dy[g], w[g], out=obuf[g]) for g in range(Gn)]  # noqa: E731
        else:
            x = torch.randn(Gn, M, K, device=dev).to(bf)
            dy = torch.randn(Gn, M, Nn, device=dev).to(bf)
            gw = torch.zeros(Gn, K, Nn, device=dev)
            fn = lambda: G.linear_wgrad_grouped(x, dy, gw)  # noqa: E731
            torch_fn = lambda: [G.linear_wgrad(x[g], dy[g], gw[g]) for g in range(Gn)]  # noqa: E731
        flops = 2.0 * Gn * M * Nn * K
        nbytes = 2.0 * Gn * (M * K + K * Nn + M * Nn)
    elif a.kernel == "gemm":
        M, Nn, K = a.m, a.n, a.k
        if a.layout == "fwd":      # y[M,N] = x[M,K] @ w[K,N]
            x = torch.randn(M, K, device=dev).to(bf)
            w = torch.randn(K, Nn, device=dev).to(bf)
            bias = torch.randn(Nn, device=dev).to(bf) if a.epi != "none" else None
            out = torch.empty(M, Nn, device=dev, dtype=bf)
            aux = torch.empty(M, Nn, device=dev, dtype=bf) if a.epi == "gelu" else None
            fn = lambda: G.linear_fwd(x, w, bias, epi="gelu" if a.epi == "gelu" else "none",  # noqa: E731
                                      aux_out=aux, out=out)
            torch_fn = lambda: torch.matmul(x, w)  # noqa: E731
            nbytes = 2.0 * (M * K + K * Nn + M * Nn * (2 if aux is not None else 1))
        elif a.layout == "dgrad":  # dx[M,K] = dy[M,N] @ w[K,N]^T
            dy = torch.randn(M, Nn, device=dev).to(bf)
            w = torch.randn(K, Nn, device=dev).to(bf)
            out = torch.empty(M, K, device=dev, dtype=bf)
            fn = lambda: G.linear_dgrad(dy, w, out=out)  # noqa: E731
            torch_fn = lambda: torch.matmul(dy, w.t())  # noqa: E731
            nbytes = 2.0 * (M * Nn + K * Nn + M * K)
        else:                      # gw[K,N] += x[M,K]^T @ dy[M,N]
            x = torch.randn(M, K, device=dev).to(bf)
            dy = torch.randn(M, Nn, device=dev).to(bf)
            gw = torch.zeros(K, Nn, device=dev)
            fn = lambda: G.linear_wgrad(x, dy, gw, ksplit=a.ksplit or None)  # noqa: E731
            torch_fn = lambda: torch.matmul(x.t(), dy)  # noqa: E731
            nbytes = 2.0 * (M * K + M * Nn) + 4.0 * K * Nn
        flops = 2.0 * M * Nn * K
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        B, nh, S, dh = a.batch, a.heads, a.seq, a.dh
        H = nh * dh
        qkv = torch.randn(B * S, 3 * H, device=dev).to(bf)
        q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
        if a.attn_poly is not None:
            A.FWD_POLY = a.attn_poly
        o, lse = A.attention_fwd(q, k, v, B, S, nh, dh)
        fwd_flops = 4.0 * B * nh * S * S * dh / 2
        if a.kernel == "attn_fwd":
            fn = lambda: A.attention_fwd(q, k, v, B, S, nh, dh)  # noqa: E731
            flops = fwd_flops
            nbytes = 2.0 * 4 * B * S * H
        else:
            do = torch.randn(B * S, H, device=dev).to(bf)
            dqkv = torch.empty(B * S, 3 * H, device=dev, dtype=bf)
            fn = lambda: A.attention_bwd(do, q, k, v, o, lse, B, S, nh, dh, dqkv=dqkv)  # noqa: E731
            flops = 2.5 * fwd_flops
            nbytes = 2.0 * 8 * B * S * H
        if a.compare_torch:
            qq = q.reshape(B, S, nh, dh).transpose(1, 2)
            kk = k.reshape(B, S, nh, dh).transpose(1, 2)
            vv = v.reshape(B, S, nh, dh).transpose(1, 2)
            torch_fn = lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True)  # noqa: E731
    elif a.kernel in ("norm_fwd", "norm_bwd"):
        T, H = a.tokens, a.hidden
        x = torch.randn(T, H, device=dev).to(bf)
        g = torch.ones(H, device=dev, dtype=bf)
        b = torch.zeros(H, device=dev, dtype=bf)
        y, mean, rstd = N.norm_fwd(x, g, b, 1e-5)
        if a.kernel == "norm_fwd":
            fn = lambda: N.norm_fwd(x, g, b, 1e-5)  # noqa: E731
            nbytes = 2.0 * 2 * T * H
        else:
            dy = torch.randn(T, H, device=dev).to(bf)
            dres = torch.randn(T, H, device=dev).to(bf)
            dg, db = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
            fn = lambda: N.norm_bwd(dy, x, g, mean, rstd, dg, db, dres)  # noqa: E731
            nbytes = 2.0 * 4 * T * H
    elif a.kernel in ("rmsnorm_fwd", "rmsnorm_bwd"):
        T, H = a.tokens, a.hidden
        x = torch.randn(T, H, device=dev).to(bf)
        g = torch.ones(H, device=dev, dtype=bf)
        y, _, rstd = N.norm_fwd(x, g, None, 1e-6, True)
        if a.kernel == "rmsnorm_fwd":
            fn = lambda: N.norm_fwd(x, g, None, 1e-6, True)  # noqa: E731
            nbytes = 2.0 * 2 * T * H
        else:
            dy = torch.randn(T, H, device=dev).to(bf)
            dres = torch.randn(T, H, device=dev).to(bf)
            dg = torch.zeros(H, device=dev)
            fn = lambda: N.norm_bwd(dy, x, g, None, rstd, dg, None, dres, True)  # noqa: E731
            nbytes = 2.0 * 4 * T * H
    elif a.kernel == "rope":
        T, nh, dh = a.tokens, a.heads, a.dh
        x = torch.randn(T, 3 * nh * dh, device=dev).to(bf)
        fn = lambda: E.rope_(x, 2 * nh, dh, a.seq)  # noqa: E731
        nbytes = 2.0 * 2 * T * 2 * nh * dh
    elif a.kernel == "softmax":
        T, V = a.tokens, a.vocab
        x = torch.randn(T, V, device=dev)
        fn = lambda: E.softmax_rows(x)  # noqa: E731
        nbytes = 4.0 * 2 * T * V
    elif a.kernel in ("swiglu", "gelu"):
        T, I = a.tokens, a.n
        if a.kernel == "swiglu":
            gu = torch.randn(T, 2 * I, device=dev).to(bf)
            fn = lambda: E.swiglu_fwd(gu)  # noqa: E731
            nbytes = 2.0 * 3 * T * I
        else:
            u = torch.randn(T, I, device=dev).to(bf)
            fn = lambda: E.gelu_fwd(u)  # noqa: E731
            nbytes = 2.0 * 2 * T * I
    elif a.kernel == "embed":
        T, H, V = a.tokens, a.hidden, a.vocab
        table = torch.randn(V, H, device=dev).to(bf)
        ids = torch.randint(0, V, (T,), device=dev)
        pe = E.sinusoid_table(a.seq, H, dev)
        fn = lambda: E.embed_fwd(ids, table, pe, a.seq)  # noqa: E731
        nbytes = 2.0 * 2 * T * H + 4.0 * T * H
    elif a.kernel == "moe_route":
        from ..ops import moe as M
        T = a.tokens
        logits = torch.randn(T, 8, device=dev)
        fn = lambda: M.route(logits, 2, 1280 * (T // 4096 or 1))  # noqa: E731
        nbytes = 4.0 * T * 8 * 2
    elif a.kernel == "allreduce_local":
        # the one-shot all-reduce (+ residual + RMSNorm) with both "ranks" on this GPU
        import ctypes
        from ..ops import _lib
        B, H = a.batch, a.hidden
        parts = [torch.randn(B, H, device=dev).to(bf) for _ in range(2)]
        resid = torch.randn(B, H, device=dev).to(bf)
        scale = torch.ones(H, device=dev, dtype=bf)
        flags = [torch.full((2,), 1 << 40, dtype=torch.int64, device=dev) for _ in range(2)]
        state = torch.zeros(2, dtype=torch.int64, device=dev)
        xo, no = torch.empty(B, H, device=dev, dtype=bf), torch.empty(B, H, device=dev, dtype=bf)
        pp = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in parts])
        fp = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in flags])
        st = _lib.status_buffer(torch.device(dev))

        def fn():
            _lib.lib().cb_ar_resid_norm(pp, fp, _lib.ptr(flags[0]), _lib.ptr(state), _lib.ptr(resid),
                                        _lib.ptr(xo), _lib.ptr(scale), _lib.ptr(None), _lib.ptr(no),
                                        2, 0, B, H, 1, ctypes.c_float(1e-6),
                                        ctypes.c_ulonglong(int(1e9)), _lib.ptr(st), _lib.stream_ptr())
        nbytes = 2.0 * 5 * B * H
    elif a.kernel == "cross_entropy":
        T, V = a.tokens, a.vocab
        logits = torch.randn(T, V, device=dev).to(bf)
        tgt = torch.randint(0, V, (T,), device=dev)
        fn = lambda: E.cross_entropy_fwd_bwd(logits, tgt, 1.0 / T)  # noqa: E731
        nbytes = 2.0 * 2 * T * V     # one read (the second pass hits L2 per row) + one write
    elif a.kernel == "adamw":
        n = a.numel
        p, m, v, g = (torch.randn(n, device=dev) for _ in range(4))
        v.abs_()
        pb = torch.empty(n, device=dev, dtype=bf)
        fn = lambda: E.adamw_step(p, m, v, g, pb, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,  # noqa: E731
                                  weight_decay=0.1, step=3)
        nbytes = n * (16.0 + 12.0 + 2.0)
    elif a.kernel == "kv_write":        # prefill-sized append of K and V into the pages
        B, nh, dh, S = a.batch, a.heads, a.dh, a.seq
        pages = (S + D.PAGE - 1) // D.PAGE
        kc = torch.zeros(B * pages, D.PAGE, nh, dh, device=dev, dtype=bf)
        vc = torch.zeros_like(kc)
        pt = torch.arange(B * pages, device=dev, dtype=torch.int32).view(B, pages)
        kv = torch.randn(B * S, 2 * nh * dh, device=dev).to(bf)
        k, v = kv[:, :nh * dh], kv[:, nh * dh:]
        pos0 = torch.zeros(B, device=dev, dtype=torch.int32)
        fn = lambda: D.kv_write(k, v, kc, vc, pt, pos0, S, nh, dh)  # noqa: E731
        nbytes = 2.0 * 2 * 2 * B * S * nh * dh
    elif a.kernel == "argmax":
        B, V = a.batch, a.vocab
        logits = torch.randn(B, V, device=dev).to(bf)
        fn = lambda: D.argmax_rows(logits)  # noqa: E731
        nbytes = 2.0 * B * V
    elif a.kernel == "normal_init":
        p = torch.empty(a.numel, device=dev)
        fn = lambda: E.normal_init_(p, seed=1234, std=0.02)  # noqa: E731
        nbytes = 4.0 * a.numel
    elif a.kernel == "colsum":           # bias gradient: column sums of a [tokens, n] matrix
        T, C = a.tokens, a.n
        x = torch.randn(T, C, device=dev).to(bf)
        acc = torch.zeros(C, device=dev)
        fn = lambda: E.colsum_into(x, acc)  # noqa: E731
        nbytes = 2.0 * T * C
    elif a.kernel in ("moe_gather", "moe_combine"):
        from ..ops import moe as M
        T, H, Ex, K = a.tokens, a.hidden, 8, 2
        C = (int(1.25 * T * K / Ex) + 127) // 128 * 128
        x = torch.randn(T, H, device=dev).to(bf)
        expert, w, _, slot, _ = M.route(torch.randn(T, Ex, device=dev), K, C)
        buf = torch.zeros(Ex * C, H, device=dev, dtype=bf)
        if a.kernel == "moe_gather":
            fn = lambda: M.gather_rows(x, expert, slot, buf, C)  # noqa: E731
            nbytes = 2.0 * (T * H + T * K * H)
        else:
            M.gather_rows(x, expert, slot, buf, C)
            fn = lambda: M.combine_rows(buf, expert, slot, C, w, x)  # noqa: E731
            nbytes = 2.0 * (T * K * H + 2 * T * H)
    else:
        B, nh, dh, S = a.batch, a.heads, a.dh, a.seq
        pages = (S + D.PAGE - 1) // D.PAGE
        kc = torch.randn(B * pages, D.PAGE, nh, dh, device=dev).to(bf)
        vc = torch.randn(B * pages, D.PAGE, nh, dh, device=dev).to(bf)
        pt = torch.arange(B * pages, device=dev, dtype=torch.int32).view(B, pages)
        ctx = torch.full((B,), S, device=dev, dtype=torch.int32)
        q = torch.randn(B, nh * dh, device=dev).to(bf)
        fn = lambda: D.decode_attention(q, kc, vc, pt, ctx, nh, dh)  # noqa: E731
        nbytes = 2.0 * 2 * B * S * nh * dh
    ms = timeit(fn, a.warmup, a.iters, a.flush_l2)
    out = {"kernel": a.kernel, "ms": round(ms, 4), "peaks": src}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_of_bf16_peak"] = round(flops / ms / 1e9 / tf, 3)
    if nbytes:
        out["gbs"] = round(nbytes / ms / 1e6, 1)
        out["frac_of_hbm_peak"] = round(nbytes / ms / 1e6 / hbm, 3)
    if a.compare_torch and torch_fn is not None:
        tms = timeit(torch_fn, a.warmup, a.iters, a.flush_l2)
        out["per_group_launch_ms" if a.kernel == "gemm" and a.groups > 1 else "torch_ms"] = \
            round(tms, 4)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
