"""Sampling parameters of a request, with AxiomOperator/rllm's names, meanings and defaults
(crates/rllm-model/src/sampler.rs:3-15; request parameters crates/rllm-server/src/engine.rs:43-75):
temperature <= 0 is greedy (argmax, first index on ties), top_k 0 and top_p 1.0 are off."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0: no limit)")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1] (1.0: no limit)")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0
