"""Pre-norm residual block: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(engine/src/model.c:906-972)."""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.manager import LayerCacheView
from .base import Block, FeedForward, Mixer, Norm, StepContext


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def tensors(self):
        return self.mixer_norm.tensors() + self.mixer.tensors() + self.ffn_norm.tensors() + self.ffn.tensors()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCacheView], write_cache: bool = True) -> None:
        if self.mixer.fuses_norm(self.mixer_norm, ctx):
            self.mixer.forward(x, ctx, cache, x, write_cache, norm=self.mixer_norm)
        else:
            self.mixer.forward(self.mixer_norm.forward(x, ctx, "block.xn"), ctx, cache, x, write_cache)
        if self.ffn.fuses_norm(self.ffn_norm, ctx):
            self.ffn.forward(x, ctx, x, norm=self.ffn_norm)
        else:
            self.ffn.forward(self.ffn_norm.forward(x, ctx, "block.xn"), ctx, x)
