"""SwiGLU feed-forward: y = W_down (silu(W_gate xn) * (W_up xn)), added into the residual stream
(engine/src/model.c:962-972; silu(g) = g / (1 + exp(-g)), engine/src/ops.c:283-288).
The gate and up matrices are stacked by rows so that one product reads xn once."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, StepContext


class SwiGLU(FeedForward):
    def __init__(self, hidden: int, intermediate: int, w_gate_up: torch.Tensor, w_down: torch.Tensor):
        if w_gate_up.shape != (2 * intermediate, hidden) or w_down.shape != (hidden, intermediate):
            raise ValueError("feed-forward weights do not fit the sizes")
        self.hidden, self.intermediate = hidden, intermediate
        self.w_gate_up, self.w_down = w_gate_up.contiguous(), w_down.contiguous()

    def tensors(self):
        return [self.w_gate_up, self.w_down]

    def fuses_norm(self, norm, ctx: StepContext) -> bool:
        return norm.as_rms() is not None and ops.fused_norm_takes(ctx.dtype, ctx.num_tokens, self.hidden, 2 * self.intermediate)

    def forward(self, xn: torch.Tensor, ctx: StepContext, residual: torch.Tensor, norm=None) -> None:
        T = ctx.num_tokens
        ws = ctx.workspace
        act_buf = ws.rows("ffn.act", T, self.intermediate, ctx.dtype)
        if norm is not None:
            # few rows: norm, gate and up, and silu(gate) * up in one launch
            nw, eps = norm.as_rms()
            act = ops.linear_skinny(xn, self.w_gate_up, act_buf, ops.EPI_SWIGLU, norm_weight=nw, eps=eps)
        elif (xn.stride(0) % 8 == 0 and xn.data_ptr() % 16 == 0
              and ops.skinny_takes(ctx.dtype, T, self.hidden, 2 * self.intermediate)):
            # a few dozen rows: the norm ran once for all of them; gate, up and silu(gate) * up in one launch
            act = ops.linear_skinny(xn, self.w_gate_up, act_buf, ops.EPI_SWIGLU)
        elif T > ops.SKINNY_MAX_ROWS and self.intermediate % 8 == 0 and ops.tcgen05_takes(xn, self.w_gate_up):
            # prompt-sized batch in bfloat16: gate, up and silu(gate) * up in one tcgen05 kernel
            act = ops.linear_tcgen05_swiglu(xn, self.w_gate_up, act_buf)
        else:
            gu = ops.linear(xn, self.w_gate_up, ws.rows("ffn.gu", T, 2 * self.intermediate, ctx.dtype), ops.LINEAR_SAME)
            act = ops.silu_mul(gu, act_buf)
        ops.linear(act, self.w_down, residual, ops.LINEAR_ACC_F32)
