"""Interfaces of the parts a decoder is put together from, and what a part sees of a step.

A part knows its own sizes and constants and nothing about the model it is in.
The residual stream is float32 [tokens, hidden]; a norm reads it and writes the
compute dtype (float32 or bfloat16); a mixer or feed-forward reads normed
activations and ADDS its result into the residual stream, so that a kernel may
do the sum in its epilogue (float32 either way).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheSpec, LayerCacheView


class Workspace:
    """Named device buffers, made once at their largest size and handed out as views.

    Addresses never change after the first use, which is what replaying a
    captured CUDA graph needs."""

    def __init__(self, device: torch.device, max_tokens: int, max_segments: int = 0, max_context: int = 0):
        self.device = device
        self.max_tokens = max_tokens
        self.max_segments = max_segments or max_tokens     # most requests in a step
        self.max_context = max_context or 8192             # most positions a request may reach
        self._bufs: Dict[str, torch.Tensor] = {}

    def rows(self, name: str, rows: int, width: int, dtype: torch.dtype) -> torch.Tensor:
        """A [rows, width] view of the buffer `name` (rows <= max_tokens)."""
        if rows > self.max_tokens:
            raise ValueError(f"workspace {name}: {rows} rows exceed the step limit of {self.max_tokens}")
        key = f"{name}/{width}/{dtype}"
        buf = self._bufs.get(key)
        if buf is None:
            buf = torch.empty((self.max_tokens, width), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:rows]

    def flat(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A flat buffer `name` of at least numel elements; it never moves or shrinks once made (zero: it starts as zeros)."""
        key = f"{name}/flat/{dtype}"
        buf = self._bufs.get(key)
        if buf is None:
            buf = (torch.zeros if zero else torch.empty)((numel,), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        elif buf.numel() < numel:
            raise ValueError(f"workspace {name} was made for {buf.numel()} elements and {numel} are asked for")
        return buf[:numel]


@dataclass
class GroupMeta:
    """Per page group: where each token's keys and values go, and each segment's block table."""
    slot_mapping: torch.Tensor      # int32 [T]: page * page_size + offset
    block_tables: torch.Tensor      # int32 [S, max_blocks]
    max_blocks: int


@dataclass
class StepContext:
    """One batch: S segments (request, its next tokens), T tokens in all, flat and in segment order."""
    num_tokens: int
    num_segments: int
    dtype: torch.dtype                       # compute dtype
    tokens: torch.Tensor                     # int32 [T]
    positions: torch.Tensor                  # int32 [T] position of each token in its request
    token_seg: torch.Tensor                  # int32 [T] segment of each token
    seg_starts: torch.Tensor                 # int32 [S+1] first token of each segment (cumulative)
    seg_context: torch.Tensor                # int32 [S] positions of the request after this step
    seg_slots: torch.Tensor                  # int32 [S] state slot of each segment's request
    groups: List[GroupMeta]
    caches: List[LayerCacheView]
    workspace: Workspace
    # the same on the host, for parts that plan launches per segment.  A part that reads these (or anything else of
    # a batch that is not a device array of this context) is not replayed faithfully by a captured graph and
    # must set capture_safe = False.
    host_seg_lens: Sequence[int] = ()
    host_seg_first_pos: Sequence[int] = ()
    host_seg_slots: Sequence[int] = ()
    max_seg_len: int = 0
    max_context: int = 0
    decode_only: bool = False                # every segment is a single token
    # tokens of single-token segments and of longer segments, as flat token indices (None: all tokens, in order)
    num_dec: int = 0
    dec_tokens: Optional[torch.Tensor] = None
    num_pre: int = 0
    pre_tokens: Optional[torch.Tensor] = None
    # segments longer than one token cut into tiles of up to 64 tokens: int32 [n, 4] = first token, rows,
    # position of the first token, segment
    pre_tiles: Optional[torch.Tensor] = None
    pre_tiles_big: Optional[torch.Tensor] = None     # the same cut into tiles of up to 128 tokens
    extra: dict = field(default_factory=dict)
    after_run: Optional[Callable[[int], None]] = None    # called by the decoder after each run of its schedule (tests)


class Part:
    """Common base: a part may hold device tensors and says how many bytes of weights it reads per step.

    capture_safe: whether a CUDA graph captured from one batch replays this part faithfully for any other batch
    with the same counts (tokens, segments, wanted rows, single-token segments, prompt tiles).  True means: the
    part's launches and their arguments depend only on those counts, on its own constants and on the context's
    device arrays (a padding segment of a decode batch has seg_slots -1 and slot mapping -1), and it neither
    synchronises nor allocates per batch.  A model with a part that says False is never captured."""

    capture_safe: bool = True

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors())

    def tensors(self) -> List[torch.Tensor]:
        return []


class Norm(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext, name: str, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x float32 [T, width] -> compute dtype [T or len(rows), width]."""
        raise NotImplementedError

    def as_rms(self):
        """(weight float32 [width], eps) if this norm is y = x / sqrt(mean(x^2) + eps) * weight, else None.  A part whose
        first kernel can apply such a norm itself (fuses_norm) asks this, not for a class, so that any norm of
        that form may be fused."""
        return None


class TokenInput(Part):
    """What turns a batch's token ids into the float32 residual stream."""

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """-> float32 [T, hidden]"""
        raise NotImplementedError


class LogitsOutput(Part):
    """What turns normed activations into float32 logits."""

    def forward(self, xn: torch.Tensor, ctx: StepContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """xn [R, hidden] in the compute dtype -> float32 [R, vocab] (in `out`, or a new tensor)."""
        raise NotImplementedError

    def fuses_norm(self, norm: "Norm", ctx: StepContext, rows: int) -> bool:
        """Whether forward_normed can apply `norm` itself for this many rows."""
        return False

    def forward_normed(self, x: torch.Tensor, rows: torch.Tensor, norm: "Norm", ctx: StepContext,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Either rotation tables that the mixer applies to q and k, or a change to the embeddings, or both."""

    def rotary_tables(self):
        """None, or (cos, sin, rot_dim): float32 [max_positions, rot_dim/2] tables for half-split pairs."""
        return None

    def on_embeddings(self, x: torch.Tensor, ctx: StepContext) -> None:
        """Absolute encodings add to the float32 embeddings here, in place."""


class Mixer(Part):
    """Mixes information between positions of a request (attention, or anything with a state)."""

    def cache_spec(self) -> CacheSpec:
        return None

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: Optional[LayerCacheView], residual: torch.Tensor,
                write_cache: bool = True, norm: Optional["Norm"] = None) -> None:
        """xn [T, hidden] in the compute dtype; adds the result into residual (float32 [T, hidden]).
        With `norm` (only ever passed when fuses_norm said yes) xn is the float32 residual stream itself and
        the part applies the norm in its first kernel."""
        raise NotImplementedError

    def fuses_norm(self, norm: "Norm", ctx: StepContext) -> bool:
        """Whether this part can apply `norm` itself for this batch (saves a launch and a round trip)."""
        return False


class FeedForward(Part):
    def forward(self, xn: torch.Tensor, ctx: StepContext, residual: torch.Tensor, norm: Optional["Norm"] = None) -> None:
        raise NotImplementedError

    def fuses_norm(self, norm: "Norm", ctx: StepContext) -> bool:
        return False


class Block(Part):
    """An arrangement of norms, a mixer and a feed-forward around the residual stream."""

    mixer: Mixer

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCacheView], write_cache: bool = True) -> None:
        raise NotImplementedError
