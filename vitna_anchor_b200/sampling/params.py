"""Sampling settings and the per-request random stream, as the reference has them
(vitna_sampling_t, engine/include/sampler.h:21-26; splitmix64, engine/src/sampler.c:40-49)."""
from __future__ import annotations

from dataclasses import dataclass

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0     # <= 0: greedy, the lowest id among equal maxima
    top_k: int = 0               # 0: off
    top_p: float = 1.0           # >= 1: off
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0)

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k is 0 (off) or a positive count")
        if not (self.top_p > 0.0):
            raise ValueError("top_p is in (0, 1], 1 meaning off")


class SplitMix64:
    """state += 0x9E37...; two xor-shift-multiplies; uniform = (next >> 11) * 2^-53."""

    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def uniform(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / 9007199254740992.0)
