"""A decoder as data: blocks, and the order in which they run.

`blocks` are the distinct layers (each with weights of its own).  `schedule`
is the list of runs: which block runs, which cache layer it uses and whether it
writes it.  A block may be named twice (its weights run twice, each run with a
cache layer of its own unless told otherwise), and a run may read the cache
layer that another run wrote (write_cache=False).  Cache layers are numbered
0..num_caches-1; each gets what its mixer's cache_spec() asks for.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..cache.manager import CacheSpec
from ..parts.base import Block, LogitsOutput, Norm, Part, PositionEncoding, StepContext, TokenInput


@dataclass(frozen=True)
class LayerRun:
    block: int                  # index into DecoderModel.blocks
    cache: int                  # cache layer this run uses
    write_cache: bool = True    # False: read what another run of the step wrote


class DecoderModel:
    def __init__(self, *, embedding: TokenInput, blocks: Sequence[Block], schedule: Sequence[LayerRun], final_norm: Norm,
                 lm_head: LogitsOutput, position: Optional[PositionEncoding], dtype: torch.dtype, vocab_size: int,
                 max_positions: int, config=None):
        self.embedding, self.blocks, self.schedule = embedding, list(blocks), list(schedule)
        self.final_norm, self.lm_head, self.position = final_norm, lm_head, position
        self.dtype, self.vocab_size, self.max_positions, self.config = dtype, vocab_size, max_positions, config
        n_caches = 1 + max((r.cache for r in self.schedule), default=-1)
        specs: List[CacheSpec] = [None] * n_caches
        writers = [0] * n_caches
        for run in self.schedule:
            spec = self.blocks[run.block].mixer.cache_spec()
            if specs[run.cache] is not None and specs[run.cache] != spec:
                raise ValueError(f"cache layer {run.cache} is used by mixers with different needs")
            specs[run.cache] = spec
            writers[run.cache] += bool(run.write_cache)
        for c, n in enumerate(writers):
            if specs[c] is not None and n != 1:
                raise ValueError(f"cache layer {c} has {n} writers in the schedule; it needs exactly one")
        self._cache_specs = specs

    def cache_specs(self) -> List[CacheSpec]:
        return list(self._cache_specs)

    def parts(self) -> List[Part]:
        return [self.embedding, *self.blocks, self.final_norm, self.lm_head]

    def step_weight_bytes(self) -> int:
        """Bytes of weights a decode step reads: every block as often as it runs, the output matrix once,
        and one embedding row per token (not counted)."""
        per_block = [b.weight_bytes() for b in self.blocks]
        return sum(per_block[r.block] for r in self.schedule) + self.final_norm.weight_bytes() + self.lm_head.weight_bytes()

    @property
    def capture_safe(self) -> bool:
        """Whether every part says that a captured CUDA graph replays it faithfully (Part.capture_safe)."""
        def safe(part) -> bool:
            if not getattr(part, "capture_safe", True):
                return False
            return all(safe(sub) for sub in vars(part).values() if isinstance(sub, Part))
        return all(safe(p) for p in self.parts() if p is not None) and (self.position is None or safe(self.position))

    def forward(self, ctx: StepContext, logit_rows: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run the batch; float32 logits [len(logit_rows), vocab] for the flat token indices in logit_rows
        (written into `out` when given, else into a new tensor)."""
        x = self.embedding.forward(ctx)
        if self.position is not None:
            self.position.on_embeddings(x, ctx)
        for i, run in enumerate(self.schedule):
            cache = ctx.caches[run.cache] if run.cache >= 0 else None
            self.blocks[run.block].forward(x, ctx, cache, run.write_cache)
            if ctx.after_run is not None:
                ctx.after_run(i)
        if logit_rows is None or logit_rows.shape[0] == 0:
            return None
        if self.lm_head.fuses_norm(self.final_norm, ctx, logit_rows.shape[0]):
            return self.lm_head.forward_normed(x, logit_rows, self.final_norm, ctx, out=out)
        xn = self.final_norm.forward(x, ctx, "head.xn", logit_rows)
        return self.lm_head.forward(xn, ctx, out=out)
