"""On-device sampling of a step's wanted rows: the logits stay on the GPU, only token ids come
back.  Semantics of AxiomOperator/rllm's device sampler (crates/rllm-core/src/sample.rs:19-109):
greedy argmax, or Gumbel-max over the candidates above a bisection threshold, with noise from a
hash of (seed, counter, token) so that a request's draws do not depend on its batch-mates.  The
counter is the request's length when the token is drawn (crates/rllm-server/src/engine.rs:871).
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams


def sample_rows(logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int],
                counts: Sequence = None) -> torch.Tensor:
    """logits float32 [rows, vocab] on the device -> int32 ids [rows] on the device.
    counts: per row, {token: times generated so far} (or None) for the penalties; rows whose
    parameters ask for a bias or a penalty have it added to their logits in place first."""
    rows = logits.shape[0]
    assert len(params) == rows and len(counters) == rows
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if any(p.adjusts for p in params):
        index, delta = [], []
        stride, vocab = logits.stride(0), logits.shape[1]
        for r, p in enumerate(params):
            if p.adjusts:
                for t, d in p.adjustments(counts[r] if counts is not None else None).items():
                    if 0 <= t < vocab and d != 0.0:
                        index.append(r * stride + t)
                        delta.append(d)
        if index:
            ops.logit_adjust(logits, torch.tensor(index, dtype=torch.int64).to(logits.device),
                             torch.tensor(delta, dtype=torch.float32).to(logits.device))
    if all(p.greedy for p in params):
        return ops.sample_rows(logits, out)
    dev = logits.device
    mask = (1 << 63) - 1
    temperature = torch.tensor([p.temperature for p in params], dtype=torch.float32).to(dev)
    top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(dev)
    top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32).to(dev)
    seed = torch.from_numpy(np.array([p.seed & ((1 << 64) - 1) for p in params], dtype=np.uint64).view(np.int64)).to(dev)
    counter = torch.tensor([c & mask for c in counters], dtype=torch.int64).to(dev)
    return ops.sample_rows(logits, out, temperature, top_k, top_p, seed, counter)
