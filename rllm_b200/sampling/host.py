"""Host-side sampler over a row of float32 logits: greedy, or temperature with top-k / top-p
from a SplitMix64 stream.  Semantics of AxiomOperator/rllm's host `Sampler`
(crates/rllm-model/src/sampler.rs:31-127, SplitMix64 at 407-421): greedy takes the first index
on ties and NaNs never win; top-k keeps the k largest; top-p keeps the smallest prefix (by
descending probability, renormalised over the top-k set when both are given) whose mass
reaches p; the draw walks the kept candidates in that order.
"""
from __future__ import annotations

import numpy as np

from .params import SamplingParams

_M64 = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & _M64

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        return z ^ (z >> 31)

    def next_f32(self) -> float:
        return float(np.float32(self.next_u64() >> 40) / np.float32(1 << 24))


def argmax(logits: np.ndarray) -> int:
    x = np.where(np.isnan(logits), -np.inf, logits)
    return int(np.argmax(x)) if x.size else 0


class HostSampler:
    def __init__(self, params: SamplingParams):
        self.params = params
        self.rng = SplitMix64(params.seed)

    def candidates(self, logits: np.ndarray):
        """(ids, probabilities) the draw is taken from, most likely first."""
        p = self.params
        x = np.where(np.isnan(logits), -np.inf, logits).astype(np.float32)
        w = np.exp((x - x.max()) * np.float32(1.0 / p.temperature), dtype=np.float32)
        order = np.argsort(-w, kind="stable")
        if p.top_k > 0:
            order = order[:min(p.top_k, order.size)]
        probs = w[order] / w[order].sum(dtype=np.float32) if p.top_k > 0 else w[order] / w.sum(dtype=np.float32)
        if p.top_p < 1.0:
            cum = np.cumsum(probs, dtype=np.float32)
            keep = int(np.searchsorted(cum, np.float32(p.top_p), side="left")) + 1
            order, probs = order[:keep], probs[:keep]
        return order, probs

    def sample(self, logits, counts=None) -> int:
        """counts: {token: times generated so far} for the penalties (applied to a copy of the row)."""
        logits = np.asarray(logits, dtype=np.float32)
        p = self.params
        if p.adjusts:
            logits = logits.copy()
            for t, d in p.adjustments(counts).items():
                if 0 <= t < logits.size:
                    logits[t] += np.float32(d)
        if p.greedy:
            return argmax(logits)
        clean = np.where(np.isnan(logits), -np.inf, logits)
        if not np.isfinite(clean.max()):
            return argmax(clean)
        ids, probs = self.candidates(clean)
        r = self.rng.next_f32() * float(probs.sum(dtype=np.float32))
        for i, pr in zip(ids, probs):
            r -= float(pr)
            if r <= 0.0:
                return int(i)
        return int(ids[-1])
