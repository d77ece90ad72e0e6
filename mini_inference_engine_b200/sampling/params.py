"""Sampling options of a request: ``SamplingParams`` of inference_engine/sampling.py:6-10
(``max_tokens``, ``temperature`` with 0 = greedy, ``ignore_eos``) plus ``seed``; the reference
draws from torch's global generator, unseeded, so its sampled runs cannot be repeated."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 0.0        # 0 = greedy
    ignore_eos: bool = False        # keep generating past EOS (fixed-length benchmarks)
    seed: int | None = None         # None = the engine's seed

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
