"""A batch's arrays: from (request, its next tokens) to what the parts and kernels read on the device.

Everything a step's kernels need besides weights and the cache is laid out in ONE pinned host buffer and copied to
the device in one piece.  Where each array lies depends only on the step's counts (tokens, segments, wanted rows,
single-token segments, prompt tiles, width of the block tables), so a CUDA graph captured for one batch finds the
arrays of any other batch with the same counts in the same places.

The step function owns one builder; tests of single parts make their own over a cache manager of theirs, so that
they see the same layout the step function produces.
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import UNMAPPED
from ..parts.base import GroupMeta, StepContext, Workspace


class MetaOverflow(RuntimeError):
    """The step's arrays do not fit the metadata buffer."""


class _Staging:
    """A pinned host buffer and the event that tells when its last copy to the device is done."""

    def __init__(self, n: int, pinned: bool):
        self.host = torch.empty(n, dtype=torch.int32, pin_memory=pinned)
        self.np = self.host.numpy()
        self.event: Optional[torch.cuda.Event] = None


def meta_words(max_tokens: int, max_segments: int, max_blocks: int, n_groups: int) -> int:
    """The most 32-bit words a step's arrays can take, from the same terms build() puts:
    tokens, positions, token_seg (3T); seg_starts (S+1); seg_context, seg_slots (2S); wanted rows (<= T);
    single-token list (<= S) and the list of the other tokens (<= T); alignment (3); tiles of 64 and of 128
    tokens, four words each (a segment of n tokens makes ceil(n/64) <= n/64 + 1 tiles); and per page group
    the slot mapping (T) and the block tables (S * max_blocks)."""
    T, S = max_tokens, min(max_segments, max_tokens)
    tiles64, tiles128 = T // 64 + S, T // 128 + S
    return 3 * T + (S + 1) + 2 * S + T + S + T + 3 + 4 * tiles64 + 4 * tiles128 + n_groups * (T + S * max_blocks)


def words_used(lens: Sequence[int], wanted: int, max_blocks: int, n_groups: int) -> int:
    """The words build() puts for segments of these lengths with `wanted` rows in all and block tables `max_blocks` wide
    (the same terms in the same order; tests hold it against meta_words)."""
    T, S = sum(lens), len(lens)
    dec = sum(1 for n in lens if n == 1)
    pre = sum(n for n in lens if n > 1)
    off = 3 * T + (S + 1) + 2 * S + wanted + dec + (pre if dec else 0)
    off = (off + 3) & ~3
    off += 4 * sum(-(-n // 64) for n in lens if n > 1) + 4 * sum(-(-n // 128) for n in lens if n > 1)
    return off + n_groups * (T + S * max_blocks)


class ContextBuilder:
    def __init__(self, cache: CacheManager, dtype: torch.dtype, workspace: Workspace, *, max_batch_tokens: int,
                 max_segments: int, max_model_len: int, device):
        self.cache, self.dtype, self.workspace = cache, dtype, workspace
        self.device = torch.device(device)
        self.page_size = cache.page_size
        self.max_model_len = max_model_len
        self.max_blocks = -(-max_model_len // self.page_size)
        self.max_segments = max_segments
        n_groups = len(cache.groups)
        decode_words = 7 * max_segments + 1 + n_groups * (max_segments + max_segments * self.max_blocks)
        self.meta_len = max(meta_words(max_batch_tokens, max_segments, self.max_blocks, n_groups), decode_words) + 8
        self._staging = [_Staging(self.meta_len, True) for _ in range(4)]
        self._turn = 0
        self.meta_dev = torch.zeros(self.meta_len, dtype=torch.int32, device=self.device)

    @property
    def turn(self) -> int:
        """Which of the staging buffers the latest build used (callers keep side buffers in step with it)."""
        return self._turn

    def _next_staging(self) -> _Staging:
        st = self._staging[self._turn]
        self._turn = (self._turn + 1) % len(self._staging)
        if st.event is not None:
            st.event.synchronize()
        return st

    def _send(self, st: _Staging, words: int) -> None:
        self.meta_dev[:words].copy_(st.host[:words], non_blocking=True)
        if st.event is None:
            st.event = torch.cuda.Event()
        st.event.record()

    # -- any mixture of segments ---------------------------------------------------------------------
    def build(self, segments: Sequence[Tuple[Hashable, Sequence[int], Sequence[int]]], fixed_blocks: Optional[int] = None,
              for_graph: bool = False) -> Tuple[StepContext, Optional[torch.Tensor]]:
        """segments: (request id, its next tokens, wanted places among them).  The requests' pages for the new
        positions must be reserved already.  Returns the context and the flat indices of the wanted rows."""
        S = len(segments)
        ps = self.page_size
        tables = self.cache.tables
        lens = [len(t) for _, t, _ in segments]
        T = sum(lens)
        R = sum(len(w) for _, _, w in segments)
        first = [tables.get(rid).length for rid, _, _ in segments]
        slots = [tables.get(rid).slot for rid, _, _ in segments]
        context = [f + n for f, n in zip(first, lens)]
        maxb = fixed_blocks or max(1, max(-(-c // ps) for c in context))

        st = self._next_staging()
        buf = st.np
        off = 0

        def put(values, count) -> slice:
            nonlocal off
            if off + count > self.meta_len:
                raise MetaOverflow(f"the step's arrays need more than the {self.meta_len} words of the metadata buffer")
            sl = slice(off, off + count)
            buf[sl] = values
            off += count
            return sl

        seg_starts = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(lens, out=seg_starts[1:])
        s_tokens = put(np.concatenate([np.asarray(t, dtype=np.int32) for _, t, _ in segments]), T)
        s_pos = put(np.concatenate([np.arange(f, f + n, dtype=np.int32) for f, n in zip(first, lens)]), T)
        s_seg = put(np.repeat(np.arange(S, dtype=np.int32), lens), T)
        s_starts = put(seg_starts, S + 1)
        s_ctx = put(np.asarray(context, dtype=np.int32), S)
        s_slots = put(np.asarray(slots, dtype=np.int32), S)
        rows = [int(seg_starts[i]) + int(w) for i, (_, _, want) in enumerate(segments) for w in want]
        s_rows = put(np.asarray(rows, dtype=np.int32), R) if R else slice(off, off)
        dec = [int(seg_starts[i]) for i in range(S) if lens[i] == 1]
        pre = [t for i in range(S) if lens[i] > 1 for t in range(int(seg_starts[i]), int(seg_starts[i + 1]))]
        s_dec = put(np.asarray(dec, dtype=np.int32), len(dec)) if dec else None
        s_pre = put(np.asarray(pre, dtype=np.int32), len(pre)) if pre and dec else None
        # tiles in the order of the keys they walk over, longest walk LAST (the kernels start from the end of the list):
        # a launch ends sooner when its longest blocks start first, and in a batch of several prompts the longest walks
        # are not those of the last prompt
        tiles = [(int(seg_starts[i]) + o, min(64, lens[i] - o), first[i] + o, i)
                 for i in range(S) if lens[i] > 1 for o in range(0, lens[i], 64)]
        tiles.sort(key=lambda t: t[2] + t[1])
        off = (off + 3) & ~3                                   # 16-byte alignment for what follows
        s_tiles = put(np.asarray(tiles, dtype=np.int32).reshape(-1), 4 * len(tiles)) if tiles else None
        big = [(int(seg_starts[i]) + o, min(128, lens[i] - o), first[i] + o, i)
               for i in range(S) if lens[i] > 1 for o in range(0, lens[i], 128)]
        big.sort(key=lambda t: t[2] + t[1])
        s_big = put(np.asarray(big, dtype=np.int32).reshape(-1), 4 * len(big)) if big else None
        group_slices = []
        for g in range(len(self.cache.groups)):
            bt = np.zeros((S, maxb), dtype=np.int32)
            sm = np.empty(T, dtype=np.int32)
            for i, (rid, _, _) in enumerate(segments):
                blocks = tables.get(rid).tables[g].blocks
                row = np.asarray(blocks[:maxb], dtype=np.int32)
                pos = np.arange(first[i], first[i] + lens[i])
                sm[seg_starts[i]:seg_starts[i + 1]] = row[pos // ps] * ps + pos % ps
                row = np.where(row == UNMAPPED, 0, row)      # pages behind a window are never read
                bt[i, :len(row)] = row
            group_slices.append((put(sm, T), put(bt.reshape(-1), S * maxb)))
        self._send(st, off)

        dev = self.meta_dev
        groups = [GroupMeta(dev[a], dev[b].view(S, maxb), maxb) for a, b in group_slices]
        ctx = StepContext(
            num_tokens=T, num_segments=S, dtype=self.dtype, tokens=dev[s_tokens], positions=dev[s_pos],
            token_seg=dev[s_seg], seg_starts=dev[s_starts], seg_context=dev[s_ctx], seg_slots=dev[s_slots], groups=groups,
            caches=self.cache.views, workspace=self.workspace, host_seg_lens=lens, host_seg_first_pos=first,
            host_seg_slots=slots, max_seg_len=max(lens), max_context=self.max_model_len if for_graph else max(context),
            decode_only=all(n == 1 for n in lens),
            num_dec=len(dec), dec_tokens=None if (s_dec is None or not pre) else dev[s_dec],
            num_pre=len(pre), pre_tokens=None if s_pre is None else dev[s_pre],
            pre_tiles=None if s_tiles is None else dev[s_tiles].view(-1, 4),
            pre_tiles_big=None if s_big is None else dev[s_big].view(-1, 4))
        return ctx, (dev[s_rows] if R else None)

    # -- single tokens, padded to a fixed number of segments -----------------------------------------------
    def build_decode(self, requests: Sequence[Hashable], tokens: Sequence[int], B: int, views: bool = True, reach: int = 0):
        """The context of a batch of single tokens, padded to B segments, at offsets that depend on B alone, so
        that a captured graph finds every array where it was at capture.  A padding segment has one token at
        position 0 that writes nothing (slot mapping -1, state slot -1) and reads page 0.  views=False: only fill the buffer."""
        S, ps, maxb = len(requests), self.page_size, self.max_blocks
        tables = self.cache.tables
        st = self._next_staging()
        buf = st.np
        n_groups = len(self.cache.groups)
        total = 7 * B + 1 + n_groups * (B + B * maxb)
        if total > self.meta_len:
            raise MetaOverflow(f"a decode batch of {B} needs more than the {self.meta_len} words of the metadata buffer")
        buf[:total] = 0
        o_tok, o_pos, o_seg, o_starts = 0, B, 2 * B, 3 * B
        o_ctx, o_slots, o_rows = 4 * B + 1, 5 * B + 1, 6 * B + 1
        o_groups = 7 * B + 1
        ar = np.arange(B + 1, dtype=np.int32)
        buf[o_seg:o_seg + B] = ar[:B]
        buf[o_starts:o_starts + B + 1] = ar
        buf[o_rows:o_rows + B] = ar[:B]
        buf[o_ctx:o_ctx + B] = 1
        buf[o_slots:o_slots + B] = -1                      # a padding segment has no state slot
        rcs = [tables.get(rid) for rid in requests]
        first = [rc.length for rc in rcs]
        buf[o_tok:o_tok + S] = [int(t) for t in tokens]
        buf[o_pos:o_pos + S] = first
        buf[o_ctx:o_ctx + S] = [f + 1 for f in first]
        buf[o_slots:o_slots + S] = [rc.slot for rc in rcs]
        for g in range(n_groups):
            o_sm = o_groups + g * (B + B * maxb)
            o_bt = o_sm + B
            buf[o_sm:o_sm + B] = -1
            bt = buf[o_bt:o_bt + B * maxb].reshape(B, maxb)
            for i, rc in enumerate(rcs):
                blocks = rc.tables[g].blocks
                row = np.asarray(blocks, dtype=np.int32)
                buf[o_sm + i] = row[first[i] // ps] * ps + first[i] % ps
                np.maximum(row, 0, out=row)
                bt[i, :len(row)] = row
        self._send(st, total)
        if not views:               # a replay needs the arrays in place, not their description
            return None, None
        dev = self.meta_dev
        groups = []
        for g in range(n_groups):
            o_sm = o_groups + g * (B + B * maxb)
            groups.append(GroupMeta(dev[o_sm:o_sm + B], dev[o_sm + B:o_sm + B + B * maxb].view(B, maxb), maxb))
        ctx = StepContext(
            num_tokens=B, num_segments=B, dtype=self.dtype, tokens=dev[o_tok:o_tok + B], positions=dev[o_pos:o_pos + B],
            token_seg=dev[o_seg:o_seg + B], seg_starts=dev[o_starts:o_starts + B + 1], seg_context=dev[o_ctx:o_ctx + B],
            seg_slots=dev[o_slots:o_slots + B], groups=groups, caches=self.cache.views, workspace=self.workspace,
            host_seg_lens=[1] * B, host_seg_first_pos=first + [0] * (B - S), host_seg_slots=[rc.slot for rc in rcs] + [-1] * (B - S),
            max_seg_len=1, max_context=reach or self.max_model_len, decode_only=True, num_dec=B)
        return ctx, dev[o_rows:o_rows + B]
