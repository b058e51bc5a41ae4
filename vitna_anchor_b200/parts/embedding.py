"""Token embedding and the output matrix.

x = the token's row, widened to float32, unscaled (engine/src/model.c:893-895);
logits = W_out xn in float32, where W_out is lm_head.weight or, when the model
ties them, the embedding table itself (engine/src/model.c:315-321, 975-978).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import LogitsOutput, StepContext, TokenInput


class Embedding(TokenInput):
    def __init__(self, vocab: int, hidden: int, table: torch.Tensor):
        if table.shape != (vocab, hidden):
            raise ValueError("the embedding table does not fit the sizes")
        self.vocab, self.hidden, self.table = vocab, hidden, table.contiguous()

    def tensors(self):
        return [self.table]

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.workspace.rows("x", ctx.num_tokens, self.hidden, torch.float32)
        return ops.embed_rows(self.table, ctx.tokens, x)


class LMHead(LogitsOutput):
    def __init__(self, vocab: int, hidden: int, weight: torch.Tensor):
        if weight.shape != (vocab, hidden):
            raise ValueError("the output matrix does not fit the sizes")
        self.vocab, self.hidden, self.weight = vocab, hidden, weight.contiguous()

    def tensors(self):
        return [self.weight]

    def _out(self, rows: int, out: Optional[torch.Tensor], device) -> torch.Tensor:
        if out is None:
            return torch.empty((rows, self.vocab), dtype=torch.float32, device=device)
        if out.shape != (rows, self.vocab) or out.dtype != torch.float32 or not out.is_contiguous():
            raise ValueError("the logits buffer is not a contiguous float32 [rows, vocab]")
        return out

    def forward(self, xn: torch.Tensor, ctx: StepContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """xn [R, hidden] in the compute dtype -> float32 logits [R, vocab] (in `out`, or a new tensor)."""
        return ops.linear(xn, self.weight, self._out(xn.shape[0], out, xn.device), ops.LINEAR_F32)

    def fuses_norm(self, norm, ctx: StepContext, rows: int) -> bool:
        return norm.as_rms() is not None and ops.fused_norm_takes(ctx.dtype, rows, self.hidden, self.vocab)

    def forward_normed(self, x: torch.Tensor, rows: torch.Tensor, norm, ctx: StepContext,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits of rmsnorm(x[rows]) in one launch (few rows); x is the float32 residual stream."""
        nw, eps = norm.as_rms()
        return ops.linear_skinny(x, self.weight, self._out(rows.shape[0], out, x.device), ops.EPI_F32, norm_weight=nw, eps=eps, rows=rows)
