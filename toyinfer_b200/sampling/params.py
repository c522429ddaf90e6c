"""Sampling options, with the reference's names, meanings and defaults
(include/options.h:17-20, src/options.cpp:33-35)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.6
    top_k: int = 20          # 0 or >= vocabulary: no limit
    top_p: float = 0.95      # 1.0: no limit
    seed: int = 0

    @property
    def greedy(self) -> bool:
        """The reference's rule (src/sampler.cpp:20): argmax when the temperature is
        (nearly) zero or only one candidate may be kept."""
        return abs(self.temperature) < 1e-3 or self.top_k == 1

    def check(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must not be negative, got {self.temperature}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must not be negative, got {self.top_k}")


GREEDY = SamplingParams(temperature=0.0, top_k=1, top_p=1.0)
