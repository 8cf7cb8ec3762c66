"""RMSNorm with the residual add fused in.

out = v * (1 / sqrt(mean(v^2) + eps)) * weight, v = x (+ delta); the weight multiplies
directly (no 1 + w), statistics in float32 (AxiomOperator/rllm:
crates/rllm-cpu/src/lib.rs:241-254; the fusion with the residual add is
crates/rllm-cuda/kernels/kernels.cu:794-820 and crates/rllm-model/src/qwen3.rs:202-208).
Parameters: size, eps.  Tensor: <prefix>weight [size], kept in float32.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, register_part


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    CAPTURE_SAFE = True
    TRACEABLE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = None

    def expected_tensors(self):
        return {self.prefix + "weight": ((self.size,), "norm")}

    def load(self, tensors):
        self.weight = self._to_device(tensors[self.prefix + "weight"], torch.float32)

    def deferrable(self):
        """(weight, eps) for a product kernel that prepares this norm in its epilogue (the division by
        the rms then happens in the product after it: csrc/ops.NormedRows)."""
        return self.weight, self.eps

    def forward(self, x, delta=None, rows=None, write_x=True):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=self.runtime.dtype, device=x.device)
        return ops.add_rms_norm(x, delta, self.weight, out, self.eps, rows=rows, write_x=write_x)
