"""Sampling a batch of logits rows on the device.

Each row has its own settings and its own uniform number, drawn on the host
from the request's splitmix64 stream (so a request's tokens do not depend on
what else was in the batch).  Rows that are all greedy take the argmax
kernel; otherwise one kernel handles greedy and sampled rows together.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams, SplitMix64


class Sampler:
    def __init__(self, vocab: int, max_rows: int, device):
        self.vocab, self.max_rows, self.device = vocab, max_rows, torch.device(device)
        m = max_rows
        self._out = torch.empty(m, dtype=torch.int32, device=self.device)
        # the rows' settings in one device buffer, filled by ONE copy from pinned host memory:
        # uniforms (float64), temperature, top_p (float32), top_k (int32), max_rows of each
        self._dev = torch.empty(20 * m, dtype=torch.uint8, device=self.device)
        self._f64 = self._dev[:8 * m].view(torch.float64)
        self._temp = self._dev[8 * m:12 * m].view(torch.float32)
        self._top_p = self._dev[12 * m:16 * m].view(torch.float32)
        self._top_k = self._dev[16 * m:20 * m].view(torch.int32)
        self._host = [torch.empty(20 * m, dtype=torch.uint8).pin_memory() for _ in range(4)]
        self._host_np = [h.numpy() for h in self._host]
        self._events = [None] * 4
        self._turn = 0
        self._probs = None   # scratch [max_rows, vocab], made when a sampled row first appears

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[SplitMix64]) -> List[int]:
        """One token id per row of logits [R, vocab]; draws one uniform from rngs[r] for each sampled row."""
        return self.sample_async(logits, params, rngs).tolist()

    def last_ids(self) -> torch.Tensor:
        """The device buffer sample_async writes: row r holds the id of row r of the latest call."""
        return self._out

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[SplitMix64]) -> torch.Tensor:
        R = logits.shape[0]
        if R > self.max_rows or len(params) != R:
            raise ValueError("the sampler was made for fewer rows, or settings and rows differ in number")
        out = self._out[:R]
        if all(p.greedy for p in params):
            return ops.argmax_rows(logits, out)
        if self._probs is None:
            self._probs = torch.empty(self.max_rows * self.vocab, dtype=torch.float32, device=self.device)
        m, t = self.max_rows, self._turn
        self._turn = (t + 1) % len(self._host)
        if self._events[t] is not None:
            self._events[t].synchronize()        # the copy that last used this staging buffer is done
        buf = self._host_np[t]
        buf[:8 * m].view(np.float64)[:R] = [0.0 if p.greedy else rngs[i].uniform() for i, p in enumerate(params)]
        buf[8 * m:12 * m].view(np.float32)[:R] = [p.temperature for p in params]
        buf[12 * m:16 * m].view(np.float32)[:R] = [p.top_p for p in params]
        buf[16 * m:20 * m].view(np.int32)[:R] = [p.top_k for p in params]
        self._dev.copy_(self._host[t], non_blocking=True)
        if self._events[t] is None:
            self._events[t] = torch.cuda.Event()
        self._events[t].record()
        return ops.sample_rows(logits, self._temp[:R], self._top_k[:R], self._top_p[:R], self._f64[:R], self._probs, out)
