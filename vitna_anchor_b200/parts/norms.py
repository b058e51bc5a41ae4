"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, in float32 (engine/src/kernels.c:94-111)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, StepContext


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight: torch.Tensor):
        if weight.shape != (width,):
            raise ValueError(f"RMSNorm weight is {tuple(weight.shape)}, expected ({width},)")
        self.width, self.eps = width, float(eps)
        self.weight = weight.to(torch.float32).contiguous()   # the norm's weights are float32 in both paths

    def tensors(self):
        return [self.weight]

    def as_rms(self):
        return self.weight, self.eps

    def forward(self, x: torch.Tensor, ctx: StepContext, name: str, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.workspace.rows(name, n, self.width, ctx.dtype)
        return ops.rmsnorm_rows(x, self.weight, self.eps, out, rows)
