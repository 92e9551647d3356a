"""Sampling parameters of one request.

The first four fields, their defaults and their ranges are the reference's
(somi_inference/core/sampler.py:11-25): temperature >= 0 with 0 meaning greedy
argmax, top_k == -1 (off) or > 0, top_p in (0, 1], repetition_penalty > 0.
`seed` is an addition: the reference draws from the global generator
(sampler.py:172-173); here every request has its own counter-based stream, so
its tokens do not depend on what else is in the batch.  None picks a seed at
random when the request is made.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int | None = None

    def __post_init__(self) -> None:
        if not self.temperature >= 0.0:
            raise ValueError("temperature must be >= 0.0")
        if not (self.top_k == -1 or self.top_k > 0):
            raise ValueError("top_k must be -1 or > 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0.0, 1.0]")
        if not self.repetition_penalty > 0.0:
            raise ValueError("repetition_penalty must be > 0.0")
        if self.seed is not None and not 0 <= int(self.seed) < 2 ** 64:
            raise ValueError("seed must fit in 64 bits")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
