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
        self._out = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._f32 = torch.empty(2 * max_rows, dtype=torch.float32, device=self.device)      # temperature, top_p
        self._i32 = torch.empty(max_rows, dtype=torch.int32, device=self.device)            # top_k
        self._f64 = torch.empty(max_rows, dtype=torch.float64, device=self.device)          # uniforms
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
        temp = np.array([p.temperature for p in params], dtype=np.float32)
        top_p = np.array([p.top_p for p in params], dtype=np.float32)
        top_k = np.array([p.top_k for p in params], dtype=np.int32)
        u = np.array([0.0 if p.greedy else rngs[i].uniform() for i, p in enumerate(params)], dtype=np.float64)
        self._f32[:R].copy_(torch.from_numpy(temp)); self._f32[self.max_rows:self.max_rows + R].copy_(torch.from_numpy(top_p))
        self._i32[:R].copy_(torch.from_numpy(top_k)); self._f64[:R].copy_(torch.from_numpy(u))
        return ops.sample_rows(logits, self._f32[:R], self._i32[:R], self._f32[self.max_rows:self.max_rows + R], self._f64[:R],
                               self._probs, out)
