"""The flat batch of one step.

A step holds, for each request in it, the request's next tokens: a portion of a prompt of any
length beside single decoded tokens of other requests.  The tokens of one request are
contiguous and in ascending position; `want` names the places among them whose logits are
asked for.  AxiomOperator/rllm flattens the same way (crates/rllm-model/src/lib.rs:18-35,
crates/rllm-model/src/generate.rs:85-139).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch


@dataclass
class StepItem:
    """`tokens`: the request's next token ids; `want`: indices into `tokens` (may be empty)."""
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepContext:
    """Everything a part may read about the step.  Device tensors are int32."""
    n_tokens: int
    n_requests: int
    tokens: torch.Tensor               # [n]
    positions: torch.Tensor            # [n] absolute position of each token in its request
    seq_ids: torch.Tensor              # [n] row of the token's request in this step
    cu_q: torch.Tensor                 # [R+1] start of each request's tokens in the flat batch
    ctx_lens: torch.Tensor             # [R] length of each request after this step
    logit_rows: Optional[torch.Tensor]  # [m] flat indices of the wanted tokens
    # host copies, for dispatch decisions
    q_lens: list = field(default_factory=list)
    start_pos: list = field(default_factory=list)
    ctx_lens_host: list = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_len: int = 0
    state_slots: Optional[torch.Tensor] = None   # [R] slot of each request's fixed-size state
    plans: dict = field(default_factory=dict)    # per-step scratch of the kernels' dispatchers (what depends on the step's shape only)
    scratch: dict = field(default_factory=dict)  # emptied at the start of every forward pass: results that the layers of one pass share
