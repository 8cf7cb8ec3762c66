"""Token embedding and LM head.

Embedding: x[t,:] = table[tokens[t],:] into the float32 residual stream, no scaling
(AxiomOperator/rllm: crates/rllm-model/src/qwen3.rs:191).  LM head: logits = rows . W^T in
float32, W its own tensor or, when `tied_to` names one, the embedding table
(crates/rllm-model/src/qwen3.rs:151-154, 232).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Part, register_part


@register_part("embedding", "embedding")
class Embedding(Part):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight = None

    def expected_tensors(self):
        return {self.prefix + "weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def load(self, tensors):
        self.weight = self._to_device(tensors[self.prefix + "weight"])

    def forward(self, tokens):
        out = torch.empty((tokens.numel(), self.hidden_size), dtype=torch.float32, device=tokens.device)
        return ops.embed(self.weight, tokens, out, ops.error_word(tokens.device))


@register_part("lm_head", "lm_head")
class LMHead(Part):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.weight = None

    def expected_tensors(self):
        if self.tied_to:
            return {}
        return {self.prefix + "weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def ignorable_tensors(self):
        """A tied model may still store the head; it is not read."""
        return {self.prefix + "weight"} if self.tied_to else set()

    def load(self, tensors, shared=None):
        if self.tied_to:
            self.weight = shared[self.tied_to]
        else:
            self.weight = self._to_device(tensors[self.prefix + "weight"])

    def forward(self, h):
        """h [m, hidden] normed rows -> float32 logits [m, vocab]."""
        return ops.linear(h, self.weight, out_dtype=torch.float32)
