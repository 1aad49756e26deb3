"""LayerNorm / RMSNorm forward and backward (``csrc/norm.cu``), per-token statistics in fp32.

The reference's ``math::layer_norm`` (plugins/model-transformer/src/lib.rs:105-128) normalises
over whatever slice it is handed; the model code there hands it the whole ``[S*H]`` buffer.
These ops implement the per-token operator (equal to the reference at ``S == 1``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


def norm_fwd(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float,
             rms: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
    """Returns ``(y, mean, rstd)``; ``mean`` is ``None`` for RMSNorm."""
    T, H = x.shape
    if not x.is_cuda:
        xf = x.float()
        if rms:
            rstd = torch.rsqrt((xf * xf).mean(-1) + eps)
            y = xf * rstd[:, None] * gamma.float()
            return y.to(x.dtype), None, rstd
        mean = xf.mean(-1)
        var = ((xf - mean[:, None]) ** 2).mean(-1)
        rstd = torch.rsqrt(var + eps)
        y = (xf - mean[:, None]) * rstd[:, None] * gamma.float()
        if beta is not None:
            y = y + beta.float()
        return y.to(x.dtype), mean, rstd
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    y = torch.empty_like(x)
    mean = None if rms else torch.empty(T, dtype=torch.float32, device=x.device)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    rc = _lib.lib().cb_norm_fwd(_lib.ptr(x), _lib.ptr(gamma), _lib.ptr(beta), _lib.ptr(y),
                                _lib.ptr(mean), _lib.ptr(rstd), T, H,
                                _lib.ctypes.c_float(eps), int(rms),
                                _lib.ptr(_lib.status_buffer(x.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "cb_norm_fwd")
    return y, mean, rstd


def norm_bwd(dy: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor,
             mean: Optional[torch.Tensor], rstd: torch.Tensor, dgamma: torch.Tensor,
             dbeta: Optional[torch.Tensor], dres: Optional[torch.Tensor] = None,
             rms: bool = False, colsum: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Returns ``dx (+ dres)``; accumulates into the fp32 ``dgamma`` / ``dbeta``.  With ``colsum``
    (fp32 ``[H]``) the column sums of the returned tensor are added to it as well: the result is
    the gradient of a residual stream, so these are the bias gradient of the linear layer that
    wrote into that stream, taken in the same pass."""
    T, H = x.shape
    if not x.is_cuda:
        xf, dyf, g = x.float(), dy.float(), gamma.float()
        if rms:
            xh = xf * rstd[:, None]
            dg = dyf * g
            dx = rstd[:, None] * (dg - xh * (dg * xh).mean(-1, keepdim=True))
        else:
            xh = (xf - mean[:, None]) * rstd[:, None]
            dg = dyf * g
            dx = rstd[:, None] * (dg - dg.mean(-1, keepdim=True)
                                  - xh * (dg * xh).mean(-1, keepdim=True))
            if dbeta is not None:
                dbeta.add_(dyf.sum(0))
        dgamma.add_((dyf * xh).sum(0))
        if dres is not None:
            dx = dx + dres.float()
        dx = dx.to(x.dtype)
        if colsum is not None:
            colsum.add_(dx.float().sum(0))
        return dx
    assert dy.is_contiguous() and x.is_contiguous()
    dx = torch.empty_like(x)

    def launch(cols):
        return _lib.lib().cb_norm_bwd(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(gamma), _lib.ptr(mean),
                                      _lib.ptr(rstd), _lib.ptr(dres), _lib.ptr(dx),
                                      _lib.ptr(dgamma), _lib.ptr(dbeta), _lib.ptr(cols), T, H,
                                      int(rms), _lib.ptr(_lib.status_buffer(x.device)),
                                      _lib.stream_ptr())

    rc = launch(colsum)
    if rc == -3:        # this shape runs a kernel that does not sum columns: a pass of its own
        from .elementwise import colsum_into
        rc = launch(None)
        _lib.check_rc(rc, "cb_norm_bwd")
        colsum_into(dx, colsum)
        return dx
    _lib.check_rc(rc, "cb_norm_bwd")
    return dx
