"""Rotate-half (NeoX) rotary position encoding over the whole head.

inv_freq[i] = 1 / theta^(2i / head_dim) for i < head_dim/2; the angle of pair (i, i + head_dim/2)
at position p is p * inv_freq[i], computed in float32 (AxiomOperator/rllm:
crates/rllm-cpu/src/lib.rs:256-290).  The part owns the inv_freq table; the rotation itself
is applied inside the mixer's fused kernel, which receives the table.
Parameters: head_dim, theta.  No tensors.

A position part's interface, either of:

``apply_and_store(qkv, q_norm_w, k_norm_w, eps, ctx, cache, q_out, H, K, head_dim)``: the
part itself turns the fused projection rows ``qkv`` [n, (H + 2K) * head_dim] (float32) into the
queries ``q_out`` [n, H * head_dim] and writes keys and values to ``cache`` (a PagedKVView: ``k``,
``v``, ``slots``, ``block_size``, ``write``) at the step's slots, applying the per-head q/k norm
(if the weights are given) before its own encoding; ``ctx`` is the step's StepContext (positions in
``ctx.positions``; ``ctx.scratch`` is a dictionary that lives for one forward pass, for what the
layers of the pass can share).  Any scheme can be written this way, with
kernels of its own or on top of ``ops.qk_norm_rope_store`` (which, without a table, norms and
stores without rotating).

``project_and_store(h, w_qkv, ...same arguments...) -> bool`` (optional): as apply_and_store, but the
part is given the rows before the fused projection and the projection's matrix, and may do the
projection too (one kernel with the norm, the encoding and the cache write in its epilogue); it
returns False when it does not take the step.

``table()``: for schemes of the form "rotate pairs (i, i + head_dim/2) by position * table[i]":
the float32 vector of head_dim/2 entries that the fused kernel takes; the mixer then calls the
kernel itself.  This part offers both.
"""
from __future__ import annotations

import torch

from .base import Part, PartError, register_part


@register_part("position", "rotary_neox")
class RotaryNeox(Part):
    CAPTURE_SAFE = True
    TRACEABLE = True

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

    def _angles(self, ctx):
        """(cos, sin) of the step's tokens: the same in every layer with this table, so once per pass."""
        from ..csrc import ops
        key = ("rotary_neox", self.head_dim, self.theta)
        table = ctx.scratch.get(key)
        if table is None:
            with ops.untraced():                  # once per pass, not once per layer that replays this one
                table = ctx.scratch[key] = ops.rope_table(ctx.positions, self.inv_freq)
        return table

    def apply_and_store(self, qkv, q_norm_w, k_norm_w, eps, ctx, cache, q_out, H, K, head_dim):
        from ..csrc import ops
        return ops.qk_norm_rope_store(qkv, q_norm_w, k_norm_w, None, ctx.positions, cache.slots, q_out,
                                      cache.k, cache.v, H, K, head_dim, cache.block_size, eps, write_kv=cache.write,
                                      cs_table=self._angles(ctx))

    def project_and_store(self, h, w_qkv, q_norm_w, k_norm_w, eps, ctx, cache, q_out, H, K, head_dim) -> bool:
        """Optional third form of a position part's interface: the part also does the q/k/v projection
        h . w_qkv^T itself, so that it can be one kernel with what follows it.  Returns False when it
        does not take the step (the mixer then projects and calls apply_and_store)."""
        from ..csrc import ops
        if not ops.can_fuse_qkv(h, w_qkv, head_dim, q_out, cache.k):
            return False
        ops.qkv_norm_rope_store_fused(h, w_qkv, q_norm_w, k_norm_w, self._angles(ctx), cache.slots, q_out, cache.k,
                                      cache.v, H, K, head_dim, cache.block_size, eps, write_kv=cache.write)
        return True
