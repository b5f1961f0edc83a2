"""Per-request sampling settings (the reference's `SamplingParams`,
src/sampler.rs:17-29): temperature 0 means greedy; `top_p` keeps the smallest set of
most probable tokens whose mass reaches it; `seed` starts the request's own stream of
draws, so a seeded request gives the same tokens whatever else is in its batch."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0


GREEDY = SamplingParams()
