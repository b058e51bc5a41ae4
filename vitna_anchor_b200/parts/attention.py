"""Causal grouped-query attention over the paged cache.

q = Wq xn, k = Wk xn, v = Wv xn (one product over the three matrices stacked
by rows); q and k heads are rotated by the position encoding's tables; k and v
go into the request's pages; every query reads keys 0..its own position (or
the last `window` of them) of its request; the heads are concatenated and the
output projection is added into the residual stream
(engine/src/model.c:912-959).  Query head h reads key-value head
h // (heads / kv_heads); scale = 1/sqrt(head_dim) unless given.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..cache.manager import KVSpec, LayerCacheView
from .base import Mixer, PositionEncoding, StepContext


class PagedAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, wqkv: torch.Tensor,
                 wo: torch.Tensor, position: PositionEncoding, window: int = 0, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError("heads do not divide into key-value groups")
        qd, kvd = num_heads * head_dim, num_kv_heads * head_dim
        if wqkv.shape != (qd + 2 * kvd, hidden) or wo.shape != (hidden, qd):
            raise ValueError("attention weights do not fit the head counts")
        self.hidden, self.nh, self.nkv, self.hd = hidden, num_heads, num_kv_heads, head_dim
        self.qd, self.kvd = qd, kvd
        self.wqkv, self.wo = wqkv.contiguous(), wo.contiguous()
        self.position = position
        self.window = int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(head_dim))

    def tensors(self):
        return [self.wqkv, self.wo]

    def cache_spec(self):
        return KVSpec(self.nkv, self.hd, self.window)

    def fuses_norm(self, norm, ctx: StepContext) -> bool:
        return norm.as_rms() is not None and ops.fused_norm_takes(ctx.dtype, ctx.num_tokens, self.hidden, self.qd + 2 * self.kvd)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor,
                write_cache: bool = True, norm=None) -> None:
        T = ctx.num_tokens
        ws = ctx.workspace
        meta = ctx.groups[cache.group]
        tables = self.position.rotary_tables()
        cos, sin, rot = tables if tables is not None else (None, None, 0)
        q_buf = ws.rows("att.q", T, self.qd, ctx.dtype)
        if norm is not None and rot == self.hd and write_cache:
            # few rows: norm, the three projections, the rotation and the cache write in one launch
            nw, eps = norm.as_rms()
            q = ops.linear_skinny(xn, self.wqkv, q_buf, ops.EPI_ROPE, norm_weight=nw, eps=eps,
                                  rope=(ctx.positions, cos, sin, meta.slot_mapping, cache.pages, self.nh, self.nkv, self.hd))
        elif (norm is None and rot == self.hd and write_cache and xn.stride(0) % 8 == 0 and xn.data_ptr() % 16 == 0
              and ops.skinny_takes(ctx.dtype, T, self.hidden, self.qd + 2 * self.kvd)):
            # a few dozen rows: the norm ran once for all of them; projections, rotation and cache write in one launch
            q = ops.linear_skinny(xn, self.wqkv, q_buf, ops.EPI_ROPE,
                                  rope=(ctx.positions, cos, sin, meta.slot_mapping, cache.pages, self.nh, self.nkv, self.hd))
        elif (norm is None and T > ops.SKINNY_MAX_ROWS and rot == self.hd and self.hd in (64, 128) and write_cache
              and ops.tcgen05_takes(xn, self.wqkv)):
            # prompt-sized batch in bfloat16: the projections, the rotation and the cache write in one tcgen05 kernel
            q = ops.linear_tcgen05_rope(xn, self.wqkv, q_buf, ctx.positions, cos, sin, meta.slot_mapping, cache.pages, self.nh,
                                        self.nkv, self.hd)
        else:
            qkv_buf = ws.rows("att.qkv", T, self.qd + 2 * self.kvd, ctx.dtype)
            if norm is not None:
                nw, eps = norm.as_rms()
                qkv = ops.linear_skinny(xn, self.wqkv, qkv_buf, ops.EPI_SAME, norm_weight=nw, eps=eps)
            else:
                qkv = ops.linear(xn, self.wqkv, qkv_buf, ops.LINEAR_SAME)
            q = ops.rope_store(qkv, ctx.positions, cos, sin, meta.slot_mapping, q_buf, cache.pages if write_cache else None,
                               self.nh, self.nkv, self.hd, rot, cache.pages.shape[3])
        att = ops.attention(q, cache.pages, meta, ctx, ws.rows("att.out", T, self.qd, ctx.dtype), self.nh, self.nkv,
                            self.hd, self.scale, self.window)
        ops.linear(att, self.wo, residual, ops.LINEAR_ACC_F32)
