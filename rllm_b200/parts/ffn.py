"""SwiGLU feed-forward: out = (silu(h . Wg^T) * (h . Wu^T)) . Wd^T, no biases
(AxiomOperator/rllm: crates/rllm-core/src/lib.rs:247-262, crates/rllm-cpu/src/lib.rs:292-298).
Parameters: hidden_size, intermediate_size.  Tensors: <prefix>{gate,up,down}_proj.weight.
Load-time transform: gate and up are stacked into one [2F, hidden] matrix so that one product
feeds the activation kernel.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, register_part


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    CAPTURE_SAFE = True
    TRACEABLE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def expected_tensors(self):
        F, d = self.intermediate_size, self.hidden_size
        return {self.prefix + "gate_proj.weight": ((F, d), "matrix"),
                self.prefix + "up_proj.weight": ((F, d), "matrix"),
                self.prefix + "down_proj.weight": ((d, F), "matrix")}

    def load(self, tensors):
        g = tensors[self.prefix + "gate_proj.weight"]
        u = tensors[self.prefix + "up_proj.weight"]
        self.w_gate_up = self._to_device(torch.cat([g.to(self.runtime.dtype), u.to(self.runtime.dtype)], 0))
        self.w_down = self._to_device(tensors[self.prefix + "down_proj.weight"])

    def first_product(self):
        return self.w_gate_up, True

    def last_product(self):
        return self.w_down, self.w_gate_up, True          # the down product follows the gate/up kernel

    def forward(self, h, ctx=None, residual=None, then_norm=None):
        """`h` may be ops.NormedRows; then_norm as for the attention part."""
        n = h.shape[0]
        act = torch.empty((n, self.intermediate_size), dtype=self.runtime.dtype, device=h.device)
        ops.gate_up_swiglu(h, self.w_gate_up, act)
        # the down product runs directly behind the gate/up product: ops is told so and keeps both on
        # one kernel family
        before = ops.Preceding(h.xw if isinstance(h, ops.NormedRows) else h, self.w_gate_up, swiglu=True)
        if residual is not None:
            if then_norm is not None:
                return ops.linear(act, self.w_down, out=residual, accumulate=True, then_norm=then_norm)
            ops.linear(act, self.w_down, out=residual, accumulate=True, follow=before)
            return None
        return ops.linear(act, self.w_down, out_dtype=torch.float32, follow=before)
