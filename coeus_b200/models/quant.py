"""Weight-only quantisation of a decoder's matrices: symmetric integer grids per output column
(optionally per group of input rows), applied in place as quantise -> dequantise so that every
kernel keeps running on bf16 / fp32 weights that sit exactly on the grid, plus a compact export
(int8 codes + fp16-representable scales) for storage.  This is what gives the reference's
``QuantizableModel{quantize, is_quantized}`` (src/core/model.rs:191-200, no implementor there) a
body; low-precision tensor-core GEMMs on the codes themselves are not part of it."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch

from ..foundation.error import ConfigError


@dataclass
class QuantConfig:
    bits: int = 8                 # 2..8, symmetric signed grid
    group_size: int = 0           # input rows per scale; 0 = one scale per output column
    include_embeddings: bool = False

    def validate(self) -> None:
        if not 2 <= self.bits <= 8:
            raise ConfigError.invalid("bits", self.bits, "Weight quantisation supports 2 to 8 bits")
        if self.group_size < 0:
            raise ConfigError.invalid("group_size", self.group_size, "Group size must be >= 0")


def quantize_matrix(w: torch.Tensor, bits: int, group_size: int = 0
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [in, out]`` -> ``(codes int8 [in, out], scales fp32 [groups, out])`` with
    ``w ~= codes * scales[group of the row]``."""
    qmax = float(2 ** (bits - 1) - 1)
    rows = w.shape[0]
    g = rows if group_size <= 0 or group_size >= rows else group_size
    n_groups = (rows + g - 1) // g
    wf = w.float()
    pad = n_groups * g - rows
    if pad:
        wf = torch.cat([wf, wf.new_zeros(pad, w.shape[1])], 0)
    blocks = wf.view(n_groups, g, -1)
    scales = blocks.abs().amax(1).clamp_min(1e-12) / qmax
    codes = torch.round(blocks / scales[:, None, :]).clamp_(-qmax, qmax).to(torch.int8)
    return codes.view(n_groups * g, -1)[:rows], scales


def dequantize_matrix(codes: torch.Tensor, scales: torch.Tensor, group_size: int = 0
                      ) -> torch.Tensor:
    rows = codes.shape[0]
    g = rows if group_size <= 0 or group_size >= rows else group_size
    idx = torch.arange(rows, device=codes.device) // g
    return codes.float() * scales[idx]


def quantize_model_(lm, cfg: QuantConfig) -> Dict[str, Tuple[torch.Tensor, torch.Tensor]]:
    """Snap every weight matrix of ``lm`` (a :class:`DecoderLM`) to its grid in place (master and
    working copy) and return ``name -> (codes, scales)``.  Norm scales and biases stay as they
    are; embeddings and the LM head only with ``include_embeddings``."""
    cfg.validate()
    out = {}
    for spec in lm.layout.specs:
        if spec.kind == "embed" and not cfg.include_embeddings:
            continue
        if spec.kind not in ("weight", "embed") or len(spec.shape) < 2:
            continue
        if spec.name == "output_proj" and not cfg.include_embeddings:
            continue
        w = lm.master[spec.name]
        mats = w.reshape(-1, *spec.shape[-2:])              # experts: one matrix each
        codes, scales = [], []
        for i in range(mats.shape[0]):
            c, s = quantize_matrix(mats[i], cfg.bits, cfg.group_size)
            mats[i].copy_(dequantize_matrix(c, s, cfg.group_size))
            codes.append(c)
            scales.append(s)
        out[spec.name] = (torch.stack(codes).reshape(*spec.shape[:-2], *codes[0].shape),
                          torch.stack(scales).reshape(*spec.shape[:-2], *scales[0].shape))
    lm.sync_working_copy()
    return out
