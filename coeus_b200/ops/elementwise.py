"""Memory-bound ops (``csrc/elementwise.cu``): embedding (+ sinusoidal positions), fused
softmax-cross-entropy, AdamW, GELU / SwiGLU, row softmax, RoPE, column sums, sin-init.

Every function runs the CUDA kernel for CUDA tensors and a float32 PyTorch restatement for CPU
tensors (used as the oracle by the GPU tests and by the CPU-only test tier).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _lib
from .gemm import _gelu_grad_ref, _gelu_ref

c_float = ctypes.c_float
c_size_t = ctypes.c_size_t


# ------------------------------------------------------------------------------ positions
def sinusoid_table(S: int, H: int, device) -> torch.Tensor:
    """``PE[p,2i] = sin(p / 10000^(2i/H))``, ``PE[p,2i+1] = cos(...)`` as fp32 ``[S,H]``
    (reference: plugins/model-transformer/src/lib.rs:398-414)."""
    device = torch.device(device)
    pe = torch.empty((S, H), dtype=torch.float32, device=device)
    if device.type != "cuda":
        pos = torch.arange(S, dtype=torch.float32)[:, None]
        k = torch.arange(0, H, 2, dtype=torch.float32)[None, :]
        div = torch.pow(torch.tensor(10000.0), k / H)
        pe[:, 0::2] = torch.sin(pos / div)
        pe[:, 1::2] = torch.cos(pos / div)
        return pe
    with torch.cuda.device(device):
        rc = _lib.lib().cb_sinusoid_pe(_lib.ptr(pe), S, H, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_sinusoid_pe")
    return pe


# ------------------------------------------------------------------------------ embedding
def embed_fwd(ids: torch.Tensor, table: torch.Tensor, pe: Optional[torch.Tensor], S: int,
              pos_offset: int = 0) -> torch.Tensor:
    """``out[t] = table[ids[t]] + pe[t % S + pos_offset]``; ids is a flat int64 ``[T]``."""
    T = ids.numel()
    V, H = table.shape
    if not table.is_cuda:
        out = table[ids.reshape(-1)].float()
        if pe is not None:
            pos = (torch.arange(T) % S) + pos_offset
            out = out + pe[pos]
        return out.to(table.dtype)
    ids = ids.reshape(-1).contiguous()
    assert ids.dtype == torch.int64
    out = torch.empty((T, H), dtype=torch.bfloat16, device=table.device)
    st = _lib.status_buffer(table.device)
    rc = _lib.lib().cb_embed_fwd(_lib.ptr(ids), _lib.ptr(table), _lib.ptr(pe), _lib.ptr(out), T, H,
                                 V, S, pos_offset, _lib.ptr(st), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_embed_fwd")
    return out


def embed_bwd(ids: torch.Tensor, dy: torch.Tensor, grad_table: torch.Tensor) -> None:
    """``grad_table[ids[t]] += dy[t]`` (fp32 accumulation)."""
    T = ids.numel()
    V, H = grad_table.shape
    if not dy.is_cuda:
        grad_table.index_add_(0, ids.reshape(-1), dy.float())
        return
    ids = ids.reshape(-1).contiguous()
    rc = _lib.lib().cb_embed_bwd(_lib.ptr(ids), _lib.ptr(dy), _lib.ptr(grad_table), T, H, V,
                                 _lib.stream_ptr())
    _lib.check_rc(rc, "cb_embed_bwd")


# ------------------------------------------------------------------------------ loss
def cross_entropy_fwd_bwd(logits: torch.Tensor, targets: torch.Tensor,
                          grad_scale: float, vocab: Optional[int] = None) -> torch.Tensor:
    """Per-token loss ``[T]`` (fp32); ``logits`` is overwritten by
    ``(softmax - onehot) * grad_scale``.  A negative target is ignored (loss 0, zero gradient).
    ``vocab`` (default: the full width) limits the softmax to the first ``vocab`` columns; the
    padding columns beyond it receive zero gradient."""
    T, W = logits.shape
    V = vocab if vocab is not None else W
    if not logits.is_cuda:
        if V != W:
            loss = cross_entropy_fwd_bwd(logits[:, :V], targets, grad_scale)
            logits[:, V:] = 0
            return loss
        lf = logits.float()
        lse = torch.logsumexp(lf, -1)
        tgt = targets.reshape(-1)
        valid = tgt >= 0
        safe = tgt.clamp(min=0)
        loss = (lse - lf.gather(1, safe[:, None])[:, 0]) * valid
        g = torch.softmax(lf, -1)
        g[torch.arange(T), safe] -= 1.0
        g = g * (valid[:, None] * grad_scale)
        logits.copy_(g.to(logits.dtype))
        return loss
    assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    targets = targets.reshape(-1).contiguous()
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    rc = _lib.lib().cb_cross_entropy(_lib.ptr(logits), _lib.ptr(targets), _lib.ptr(loss),
                                     _lib.ptr(None), _lib.ptr(None), T, V, logits.stride(0), 0,
                                     c_float(grad_scale), 0, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_cross_entropy")
    return loss


def cross_entropy_stats(logits: torch.Tensor, targets: torch.Tensor,
                        vocab_start: int) -> torch.Tensor:
    """Vocab-parallel half 1: per-token ``(max, sum exp(x - max), target logit or 0)`` of this
    rank's vocabulary shard, fp32 ``[T,3]``."""
    T, V = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        m = lf.max(-1).values
        s = torch.exp(lf - m[:, None]).sum(-1)
        tgt = targets.reshape(-1) - vocab_start
        inside = (tgt >= 0) & (tgt < V)
        tl = lf.gather(1, tgt.clamp(0, V - 1)[:, None])[:, 0] * inside
        return torch.stack([m, s, tl], -1)
    stats = torch.empty((T, 3), dtype=torch.float32, device=logits.device)
    targets = targets.reshape(-1).contiguous()
    rc = _lib.lib().cb_cross_entropy(_lib.ptr(logits), _lib.ptr(targets), _lib.ptr(None),
                                     _lib.ptr(stats), _lib.ptr(None), T, V, logits.stride(0),
                                     vocab_start, c_float(0.0), 1, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_cross_entropy(stats)")
    return stats


def cross_entropy_bwd_from_lse(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor,
                               vocab_start: int, grad_scale: float) -> None:
    """Vocab-parallel half 2: overwrite the shard's logits with their gradient given the
    global log-sum-exp."""
    T, V = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        g = torch.exp(lf - lse[:, None])
        tgt = targets.reshape(-1)
        loc = tgt - vocab_start
        inside = (loc >= 0) & (loc < V)
        rows = torch.arange(T)[inside]
        g[rows, loc[inside]] -= 1.0
        g = g * ((tgt >= 0)[:, None] * grad_scale)
        logits.copy_(g.to(logits.dtype))
        return
    targets = targets.reshape(-1).contiguous()
    rc = _lib.lib().cb_cross_entropy(_lib.ptr(logits), _lib.ptr(targets), _lib.ptr(None),
                                     _lib.ptr(None), _lib.ptr(lse), T, V, logits.stride(0),
                                     vocab_start, c_float(grad_scale), 2, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_cross_entropy(bwd)")


# ------------------------------------------------------------------------------ optimizer
def adamw_step(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
               p_bf16: Optional[torch.Tensor], *, lr: float, beta1: float, beta2: float,
               eps: float, weight_decay: float, step: int, grad_scale: float = 1.0,
               clip_coef: Optional[torch.Tensor] = None) -> None:
    """Decoupled-weight-decay AdamW on flat fp32 ``p/m/v`` with fp32 ``g``; refreshes the bf16
    working copy ``p_bf16`` in the same pass."""
    n = p.numel()
    if not p.is_cuda:
        gs = g * grad_scale * (float(clip_coef) if clip_coef is not None else 1.0)
        m.mul_(beta1).add_(gs, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gs, gs, value=1 - beta2)
        bc1 = 1 - beta1 ** step
        bc2 = 1 - beta2 ** step
        p.mul_(1 - lr * weight_decay).addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
        if p_bf16 is not None:
            p_bf16.copy_(p.to(p_bf16.dtype))
        return
    rc = _lib.lib().cb_adamw(_lib.ptr(p), _lib.ptr(m), _lib.ptr(v), _lib.ptr(g), _lib.ptr(p_bf16),
                             c_size_t(n), c_float(lr), c_float(beta1), c_float(beta2),
                             c_float(eps), c_float(weight_decay), step, c_float(grad_scale),
                             _lib.ptr(clip_coef), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_adamw")


def sumsq_into(g: torch.Tensor, out: torch.Tensor) -> None:
    """``out[0] += sum(g*g)`` for a flat fp32 tensor."""
    if not g.is_cuda:
        out.add_((g.float() ** 2).sum())
        return
    rc = _lib.lib().cb_sumsq(_lib.ptr(g), c_size_t(g.numel()), _lib.ptr(out), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_sumsq")


def sum_scaled_into(x: torch.Tensor, out: torch.Tensor, scale: float) -> None:
    """``out[0] += scale * sum(x)`` for a flat fp32 tensor (mean loss)."""
    if not x.is_cuda:
        out.add_(x.float().sum() * scale)
        return
    rc = _lib.lib().cb_sum_scaled(_lib.ptr(x), c_size_t(x.numel()), _lib.ptr(out),
                                  c_float(scale), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_sum_scaled")


def clip_coef_from_sumsq(sumsq: torch.Tensor, scale: float, max_norm: float,
                         coef: torch.Tensor, norm_out: Optional[torch.Tensor] = None) -> None:
    """``coef = min(1, max_norm / (sqrt(sumsq) * scale + 1e-6))`` computed on the device."""
    if not sumsq.is_cuda:
        norm = math.sqrt(float(sumsq)) * scale
        if norm_out is not None:
            norm_out.fill_(norm)
        coef.fill_(min(1.0, max_norm / (norm + 1e-6)))
        return
    rc = _lib.lib().cb_clip_coef(_lib.ptr(sumsq), c_float(scale), c_float(max_norm),
                                 _lib.ptr(coef), _lib.ptr(norm_out), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_clip_coef")


# ------------------------------------------------------------------------------ activations
def gelu_fwd(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return _gelu_ref(x.float()).to(x.dtype)
    y = torch.empty_like(x)
    rc = _lib.lib().cb_gelu_fwd(_lib.ptr(x), _lib.ptr(y), c_size_t(x.numel()), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_gelu_fwd")
    return y


def gelu_bwd(x: torch.Tensor, dy: torch.Tensor, colsum: Optional[torch.Tensor] = None
             ) -> torch.Tensor:
    """``dx = dy * gelu'(x)``.  With ``colsum`` (fp32 ``[C]``) the column sums of ``dx`` are added
    to it in the same pass: the bias gradient of the projection that produced ``x``."""
    if not x.is_cuda:
        dx = (dy.float() * _gelu_grad_ref(x.float())).to(x.dtype)
        if colsum is not None:
            colsum.add_(dx.float().sum(0))
        return dx
    dx = torch.empty_like(x)
    if colsum is not None and x.dim() == 2 and x.is_contiguous() and dy.is_contiguous():
        rc = _lib.lib().cb_gelu_bwd_colsum(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dx),
                                           _lib.ptr(colsum), x.shape[0], x.shape[1],
                                           _lib.stream_ptr())
        _lib.check_rc(rc, "cb_gelu_bwd_colsum")
        return dx
    rc = _lib.lib().cb_gelu_bwd(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dx), c_size_t(x.numel()),
                                _lib.stream_ptr())
    _lib.check_rc(rc, "cb_gelu_bwd")
    if colsum is not None:
        colsum_into(dx, colsum)
    return dx


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    """``gu`` is ``[T, 2I]`` (gate | up); returns ``silu(gate) * up`` as ``[T, I]``."""
    T, I2 = gu.shape
    I = I2 // 2
    if not gu.is_cuda:
        g, u = gu[:, :I].float(), gu[:, I:].float()
        return (torch.nn.functional.silu(g) * u).to(gu.dtype)
    y = torch.empty((T, I), dtype=gu.dtype, device=gu.device)
    rc = _lib.lib().cb_swiglu_fwd(_lib.ptr(gu), _lib.ptr(y), T, I, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_swiglu_fwd")
    return y


def swiglu_bwd(gu: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    T, I2 = gu.shape
    I = I2 // 2
    if not gu.is_cuda:
        g, u, d = gu[:, :I].float(), gu[:, I:].float(), dy.float()
        sg = torch.sigmoid(g)
        sl = g * sg
        return torch.cat([d * u * (sg + sl * (1 - sg)), d * sl], 1).to(gu.dtype)
    dgu = torch.empty_like(gu)
    rc = _lib.lib().cb_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dy), _lib.ptr(dgu), T, I,
                                  _lib.stream_ptr())
    _lib.check_rc(rc, "cb_swiglu_bwd")
    return dgu


def softmax_rows(x: torch.Tensor) -> torch.Tensor:
    """Max-subtracted row softmax in fp32 (math::softmax, lib.rs:80-88)."""
    if not x.is_cuda:
        return torch.softmax(x.float(), -1)
    x = x.float().contiguous()
    R, C = x.reshape(-1, x.shape[-1]).shape
    y = torch.empty_like(x)
    rc = _lib.lib().cb_softmax_rows(_lib.ptr(x), _lib.ptr(y), R, C, _lib.stream_ptr())
    _lib.check_rc(rc, "cb_softmax_rows")
    return y


def rope_(x: torch.Tensor, nheads: int, dh: int, S: int, pos_offset: int = 0,
          theta: float = 10000.0, inverse: bool = False,
          pos_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In-place half-split rotary embedding on a ``[T, >= nheads*dh]`` view (row pitch
    ``x.stride(0)``); position of row t is ``t % S + pos_offset``, or ``t % S + pos_dev[t // S]``
    when the int32 tensor ``pos_dev`` (first position of every sequence, on the device) is given."""
    T = x.shape[0]
    if not x.is_cuda:
        half = dh // 2
        base = pos_dev.long()[torch.arange(T) // S] if pos_dev is not None else pos_offset
        pos = ((torch.arange(T) % S) + base).float()
        inv = theta ** (-2.0 * torch.arange(half).float() / dh)
        ang = pos[:, None] * inv[None, :]
        sn, cs = torch.sin(ang)[:, None, :], torch.cos(ang)[:, None, :]
        if inverse:
            sn = -sn
        xv = x[:, :nheads * dh].reshape(T, nheads, dh).float()
        a, b = xv[..., :half], xv[..., half:]
        out = torch.cat([a * cs - b * sn, a * sn + b * cs], -1).reshape(T, nheads * dh)
        x[:, :nheads * dh] = out.to(x.dtype)
        return x
    if pos_dev is not None:
        assert pos_dev.dtype == torch.int32 and pos_dev.numel() * S >= T
        rc = _lib.lib().cb_rope_dev(_lib.ptr(x), T, nheads, dh, x.stride(0), S, _lib.ptr(pos_dev),
                                    c_float(theta), int(inverse), _lib.stream_ptr())
        _lib.check_rc(rc, "cb_rope_dev")
        return x
    rc = _lib.lib().cb_rope(_lib.ptr(x), T, nheads, dh, x.stride(0), S, pos_offset,
                            c_float(theta), int(inverse), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_rope")
    return x


def llama3_inv_freq(dh: int, theta: float, factor: float, low: float, high: float,
                    original_max: int) -> torch.Tensor:
    """Rotary frequencies with the Llama-3.1 scaling: wavelengths longer than
    ``original_max / low`` are divided by ``factor``, shorter than ``original_max / high`` kept,
    in between interpolated."""
    inv = theta ** (-2.0 * torch.arange(dh // 2).float() / dh)
    wavelen = 2 * math.pi / inv
    smooth = ((original_max / wavelen) - low) / (high - low)
    mid = (1 - smooth) * inv / factor + smooth * inv
    out = torch.where(wavelen > original_max / low, inv / factor, inv)
    is_mid = (wavelen <= original_max / low) & (wavelen >= original_max / high)
    return torch.where(is_mid, mid, out)


def rope_freq_(x: torch.Tensor, nheads: int, dh: int, S: int, inv_freq: torch.Tensor,
               pos_offset: int = 0, inverse: bool = False,
               pos_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`rope_` with an explicit frequency table (scaled rotary embeddings), written with
    tensor ops on whatever device ``x`` lives on: the hand-written kernel derives its
    frequencies from ``theta`` alone, so models with scaled frequencies take this path."""
    T = x.shape[0]
    half = dh // 2
    t = torch.arange(T, device=x.device)
    base = pos_dev.long()[t // S] if pos_dev is not None else pos_offset
    pos = ((t % S) + base).float()
    ang = pos[:, None] * inv_freq.to(x.device)[None, :]
    sn, cs = torch.sin(ang)[:, None, :], torch.cos(ang)[:, None, :]
    if inverse:
        sn = -sn
    xv = x[:, :nheads * dh].reshape(T, nheads, dh).float()
    a, b = xv[..., :half], xv[..., half:]
    x[:, :nheads * dh] = torch.cat([a * cs - b * sn, a * sn + b * cs], -1).reshape(
        T, nheads * dh).to(x.dtype)
    return x


def colsum_into(x: torch.Tensor, out: torch.Tensor) -> None:
    """``out[c] += sum_t x[t,c]`` with fp32 accumulation (bias gradients)."""
    T, C = x.shape
    if not x.is_cuda:
        out.add_(x.float().sum(0))
        return
    rc = _lib.lib().cb_colsum(_lib.ptr(x), _lib.ptr(out), T, C, x.stride(0), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_colsum")


def _philox4x32(counter_lo, counter_hi, seed: int):
    """Philox4x32-10 on numpy uint64 lanes holding 32-bit values; returns the four output words."""
    import numpy as np
    m32 = np.uint64(0xFFFFFFFF)
    c = [counter_lo & m32, counter_hi & m32, np.zeros_like(counter_lo), np.zeros_like(counter_lo)]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c[0]
        p1 = np.uint64(0xCD9E8D57) * c[2]
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & m32, p1 >> np.uint64(32), p1 & m32
        c = [hi1 ^ c[1] ^ np.uint64(k0), lo1, hi0 ^ c[3] ^ np.uint64(k1), lo0]
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return c


def normal_init_(p: torch.Tensor, seed: int, mean: float = 0.0, std: float = 0.02,
                 index_offset: int = 0) -> torch.Tensor:
    """Fill a contiguous fp32 tensor with N(mean, std) from a counter-based generator
    (Philox4x32-10 + Box-Muller): element ``i`` depends on ``(seed, index_offset + i)`` only, so
    a shard of a tensor draws the values the whole tensor would have there, on CPU and GPU alike
    (the two agree to the precision of ``logf`` / ``sincosf``).  The reference has the
    deterministic sine init only (plugins/model-transformer/src/lib.rs:604-611)."""
    n = p.numel()
    seed &= (1 << 64) - 1
    if n == 0:
        return p
    if not p.is_cuda:
        import numpy as np
        g = np.arange(index_offset // 4, (index_offset + n + 3) // 4, dtype=np.uint64)
        w = _philox4x32(g & np.uint64(0xFFFFFFFF), g >> np.uint64(32), seed)
        u = [((x >> np.uint64(8)).astype(np.float32) * np.float32(2.0 ** -24) + np.float32(2.0 ** -25))
             for x in w]
        z = np.empty((g.size, 4), dtype=np.float32)
        for h in range(2):
            r = np.sqrt(np.float32(-2.0) * np.log(u[2 * h]))
            th = np.float32(6.283185307179586) * u[2 * h + 1]
            z[:, 2 * h] = r * np.cos(th)
            z[:, 2 * h + 1] = r * np.sin(th)
        lo = index_offset - (index_offset // 4) * 4
        vals = np.float32(mean) + np.float32(std) * z.reshape(-1)[lo:lo + n]
        p.copy_(torch.from_numpy(vals).reshape(p.shape))
        return p
    assert p.dtype == torch.float32 and p.is_contiguous()
    rc = _lib.lib().cb_normal_init(_lib.ptr(p), c_size_t(n), c_size_t(index_offset),
                                   ctypes.c_uint64(seed), c_float(mean), c_float(std),
                                   _lib.stream_ptr())
    _lib.check_rc(rc, "cb_normal_init")
    return p


def sin_init_(p: torch.Tensor, hidden: int, index_offset: int = 0) -> torch.Tensor:
    """The reference's deterministic init ``clamp(sin(f32(i) * 0.1234567) * sqrt(2/H), ±0.1)``
    (plugins/model-transformer/src/lib.rs:604-611) on a flat fp32 tensor."""
    scale = math.sqrt(2.0 / hidden)
    n = p.numel()
    if not p.is_cuda:
        idx = (torch.arange(n, dtype=torch.int64) + index_offset).to(torch.float32)
        val = torch.sin(idx * torch.tensor(0.1234567, dtype=torch.float32)) * torch.tensor(
            scale, dtype=torch.float32)
        p.copy_(val.clamp_(-0.1, 0.1).reshape(p.shape))
        return p
    rc = _lib.lib().cb_sin_init(_lib.ptr(p), c_size_t(n), c_size_t(index_offset), c_float(scale),
                                _lib.stream_ptr())
    _lib.check_rc(rc, "cb_sin_init")
    return p


# ------------------------------------------------------------------------------ dropout
def dropout_threshold(p: float) -> int:
    """Dropout rates are realised in steps of 1/256: the byte threshold of rate ``p``."""
    thr = int(round(float(p) * 256.0))
    if not 0 <= thr <= 255:
        raise ValueError(f"dropout rate {p} out of range [0, 1)")
    return thr


def dropout_key(seed: int, *parts: int) -> int:
    """32-bit key of one dropout site from the run's seed and integers that name the site (step,
    layer, position in the layer, micro-batch, rank ...)."""
    x = (int(seed) * 0x9E3779B1 + 0x7F4A7C15) & 0xFFFFFFFF
    for v in parts:
        x = ((x ^ (int(v) & 0xFFFFFFFF)) * 0x85EBCA6B + 0xC2B2AE35) & 0xFFFFFFFF
        x ^= x >> 15
    return x


def _mix32(x: torch.Tensor) -> torch.Tensor:
    m = 0xFFFFFFFF
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    return x ^ (x >> 16)


def dropout_mask(rows: int, cols: int, thr: int, key: int, device="cpu",
                 row_offset: int = 0) -> torch.Tensor:
    """The keep-mask (bool ``[rows, cols]``) of the kernels' dropout function
    (``csrc/common.cuh: dropout_bits``): element ``(r, c)`` has index ``(r + row_offset) * cols +
    c``, groups of four consecutive indices share one 32-bit hash, one byte per element, dropped
    when the byte is below ``thr``."""
    r = torch.arange(row_offset, row_offset + rows, dtype=torch.int64, device=device)[:, None]
    c = torch.arange(cols, dtype=torch.int64, device=device)[None, :]
    idx = r * cols + c
    group, lane = idx >> 2, idx & 3
    h = _mix32((group & 0xFFFFFFFF) ^ _mix32(((group >> 32) & 0xFFFFFFFF) ^ (key & 0xFFFFFFFF)))
    return ((h >> (8 * lane)) & 255) >= thr


def dropout_apply(x: torch.Tensor, thr: int, key: int, out: Optional[torch.Tensor] = None
                  ) -> torch.Tensor:
    """``x * mask * 256 / (256 - thr)`` for a 2-D tensor with the mask of :func:`dropout_mask`;
    ``thr == 0`` returns ``x`` itself."""
    if thr == 0:
        return x
    rows, cols = x.shape
    if not x.is_cuda:
        keep = dropout_mask(rows, cols, thr, key, x.device)
        y = torch.where(keep, x.float() * (256.0 / (256 - thr)), torch.zeros((), device=x.device))
        y = y.to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty_like(x)
    rc = _lib.lib().cb_dropout_apply(_lib.ptr(x), x.stride(0), _lib.ptr(out), out.stride(0),
                                     c_size_t(rows), cols, thr, ctypes.c_uint(key & 0xFFFFFFFF),
                                     _lib.stream_ptr())
    _lib.check_rc(rc, "cb_dropout_apply")
    return out
