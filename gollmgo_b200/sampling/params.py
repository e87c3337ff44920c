"""Per-request sampling parameters.  Names and meanings are the reference's
SamplingParams (internal/engine/sampling.go:10-15): temperature 0 = greedy,
top_k 0 = off, top_p 0 or >= 1 = off, seed.  The reference has one set for the
whole engine; here every request carries its own."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 0.0
    seed: Optional[int] = None            # None: a seed is drawn when the request is added
    max_tokens: int = 256                 # the reference's default (internal/api/chat.go:141-144)
    ignore_eos: bool = False

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (0.0 <= self.top_p <= 1.0):
            raise ValueError("top_p must be in [0, 1]")
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 1e-9
