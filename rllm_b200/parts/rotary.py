"""Rotate-half (NeoX) rotary position encoding over the whole head.

inv_freq[i] = 1 / theta^(2i / head_dim) for i < head_dim/2; the angle of pair (i, i + head_dim/2)
at position p is p * inv_freq[i], computed in float32 (AxiomOperator/rllm:
crates/rllm-cpu/src/lib.rs:256-290).  The part owns the inv_freq table; the rotation itself
is applied inside the mixer's fused kernel, which receives the table.
Parameters: head_dim, theta.  No tensors.

A position part's interface: ``table()`` returns what the mixer's kernel needs (here the
float32 inv_freq vector of head_dim/2 entries).
"""
from __future__ import annotations

import torch

from .base import Part, PartError, register_part


@register_part("position", "rotary_neox")
class RotaryNeox(Part):
    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        if self.head_dim % 2:
            raise PartError(f"rotary_neox: head_dim {self.head_dim} must be even")
        i = torch.arange(0, self.head_dim, 2, dtype=torch.float32)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), i / self.head_dim)
        self.inv_freq = inv.to(runtime.device)

    def table(self):
        return self.inv_freq
