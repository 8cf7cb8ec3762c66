"""Sampling parameters of a request, with AxiomOperator/rllm's names, meanings and defaults
(crates/rllm-model/src/sampler.rs:3-15; request parameters crates/rllm-server/src/engine.rs:43-75):
temperature <= 0 is greedy (argmax, first index on ties), top_k 0 and top_p 1.0 are off.
`logit_bias` ((token, delta) pairs), `frequency_penalty` and `presence_penalty` are added to the
logits before anything else: for every token generated so far, c times, the logit goes down by
c * frequency_penalty + presence_penalty (crates/rllm-server/src/engine.rs:1113-1129; the
device sampler's `adjust` list, crates/rllm-core/src/sample.rs:28-29, 56-61)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    logit_bias: tuple = ()            # ((token id, delta), ...)

    def __post_init__(self):
        object.__setattr__(self, "logit_bias", tuple((int(t), float(d)) for t, d in self.logit_bias))
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0 (0: no limit)")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1] (1.0: no limit)")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def adjusts(self) -> bool:
        return bool(self.logit_bias) or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    def adjustments(self, counts=None) -> dict:
        """{token: delta} to add to the logits: the bias plus, for every token in `counts` (how
        often each token was generated so far), -(count * frequency_penalty + presence_penalty).
        Deltas of the same token are summed."""
        out: dict = {}
        for t, d in self.logit_bias:
            out[t] = out.get(t, 0.0) + d
        if counts and (self.frequency_penalty != 0.0 or self.presence_penalty != 0.0):
            for t, c in counts.items():
                out[t] = out.get(t, 0.0) - (c * self.frequency_penalty + self.presence_penalty)
        return out
