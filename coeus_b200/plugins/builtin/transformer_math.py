"""The four numeric helpers of the reference's transformer plugin with their call shapes
(plugins/model-transformer/src/lib.rs:50-128, private ``mod math`` there): flat fp32 buffers in,
flat fp32 buffers out.  CPU tensors (and plain sequences) are computed in fp32 with PyTorch; CUDA
tensors go through the framework's kernels (bf16 tensor-core GEMM, row softmax, GELU), which is
what the model's forward pass uses.

``layer_norm`` keeps the reference's definition: ONE mean and variance over the whole buffer it is
given (its callers pass all ``S x H`` values at once, lib.rs:469,488,906-911), ``scale`` and
``bias`` indexed modulo their length.  The model itself normalises per token.
"""
from __future__ import annotations

from typing import Sequence, Union

import torch

Buf = Union[torch.Tensor, Sequence[float]]


def _t(x: Buf) -> torch.Tensor:
    return x if isinstance(x, torch.Tensor) else torch.tensor(list(x), dtype=torch.float32)


def matmul(a: Buf, b: Buf, m: int, n: int, k: int) -> torch.Tensor:
    """``C[m, n] = A[m, k] @ B[k, n]`` on row-major flat buffers; returns the flat ``[m * n]``."""
    A, B = _t(a).reshape(m, k), _t(b).reshape(k, n)
    if A.is_cuda:
        from ...ops import gemm as G
        if k % 8 == 0 and n % 8 == 0:
            out = G.gemm(A.to(torch.bfloat16).contiguous(), B.to(torch.bfloat16).contiguous(),
                         b_mn=True, out_dtype=torch.float32)
            return out.reshape(-1)
    return (A.float() @ B.float()).reshape(-1)


def softmax(input: Buf) -> torch.Tensor:
    """Max-subtracted softmax of one row."""
    x = _t(input)
    if x.is_cuda and x.dtype == torch.bfloat16:
        from ...ops import elementwise as E
        return E.softmax_rows(x.reshape(1, -1)).reshape(-1)
    x = x.float()
    e = torch.exp(x - x.max())
    return e / e.sum()


def gelu(x):
    """tanh approximation with the reference's constants; accepts a float or a tensor."""
    if isinstance(x, torch.Tensor):
        if x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
            from ...ops import elementwise as E
            return E.gelu_fwd(x)
        xf = x.float()
        return 0.5 * xf * (1.0 + torch.tanh(0.7978845608028654 * xf * (1.0 + 0.044715 * xf * xf)))
    import math
    return 0.5 * x * (1.0 + math.tanh(0.7978845608028654 * x * (1.0 + 0.044715 * x * x)))


def layer_norm(input: Buf, scale: Buf, bias: Buf, eps: float) -> torch.Tensor:
    """Whole-buffer statistics (biased variance), ``scale[i % len(scale)]``,
    ``bias[i % len(bias)]``."""
    x, g, b = _t(input).float().reshape(-1), _t(scale).float().reshape(-1), \
        _t(bias).float().reshape(-1)
    n = x.numel()
    mean = x.mean()
    var = ((x - mean) ** 2).mean()
    idx = torch.arange(n, device=x.device)
    return g[idx % g.numel()] * (x - mean) / torch.sqrt(var + eps) + b[idx % b.numel()]
