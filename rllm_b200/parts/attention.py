"""Grouped-query causal attention over the paged cache.

q/k/v projections without bias, optional per-head RMSNorm on queries and keys (one weight of
head_dim entries shared by all heads, applied before the rotation), position encoding on
queries and keys, keys and values written to the cache at the step's slots, softmax(q.k *
scale) over keys pos+1-window..pos (window 0: all), output projection
(AxiomOperator/rllm: crates/rllm-model/src/qwen3.rs:195-201; attention formula
crates/rllm-cpu/src/lib.rs:389-425; q/k norm crates/rllm-core/src/lib.rs:459-476).

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm, qk_norm_eps, window,
scale.  Tensors: <prefix>{q,k,v,o}_proj.weight and, with qk_norm, <prefix>{q,k}_norm.weight.
Load-time transform: q, k and v are stacked into one [(H + 2K) * head_dim, hidden] matrix.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PagedKVNeed, PartError, register_part


@register_part("mixer", "attention")
class Attention(Mixer):
    CAPTURE_SAFE = True
    TRACEABLE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.K = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.window = int(p.get("window", 0) or 0)
        self.scale = float(p["scale"])
        if self.H % self.K:
            raise PartError(f"attention: {self.H} heads are not a multiple of {self.K} key/value heads")
        if self.hd % 16 or self.hd > 256:
            raise PartError(f"attention: head_dim {self.hd} must be a multiple of 16 and at most 256")
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    def cache_need(self):
        return PagedKVNeed(self.K, self.hd, self.window)

    def expected_tensors(self):
        d, H, K, hd, p = self.hidden_size, self.H, self.K, self.hd, self.prefix
        t = {p + "q_proj.weight": ((H * hd, d), "matrix"), p + "k_proj.weight": ((K * hd, d), "matrix"),
             p + "v_proj.weight": ((K * hd, d), "matrix"), p + "o_proj.weight": ((d, H * hd), "matrix")}
        if self.qk_norm:
            t[p + "q_norm.weight"] = ((hd,), "norm")
            t[p + "k_norm.weight"] = ((hd,), "norm")
        return t

    def load(self, tensors):
        p, dt = self.prefix, self.runtime.dtype
        self.w_qkv = self._to_device(torch.cat([tensors[p + f"{n}_proj.weight"].to(dt) for n in "qkv"], 0))
        self.w_o = self._to_device(tensors[p + "o_proj.weight"])
        if self.qk_norm:
            self.q_norm_w = self._to_device(tensors[p + "q_norm.weight"], torch.float32)
            self.k_norm_w = self._to_device(tensors[p + "k_norm.weight"], torch.float32)

    # A norm between two products may go without a kernel of its own (ops.NormedRows): the block asks the
    # parts on both sides for the matrices of their last and first product.
    def first_product(self):
        return self.w_qkv, False

    def last_product(self):
        return self.w_o, None, False

    def forward(self, h, ctx, cache, position, residual=None, then_norm=None):
        """`h` may be ops.NormedRows; then_norm = (weight, eps): the output product also prepares the
        norm that follows and the rows come back as ops.NormedRows (needs `residual`)."""
        n = h.shape[0]
        dt = self.runtime.dtype
        q = torch.empty((n, self.H * self.hd), dtype=dt, device=self.w_qkv.device)
        whole = getattr(position, "project_and_store", None)
        if whole is not None and whole(h, self.w_qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, ctx, cache, q,
                                       self.H, self.K, self.hd):
            qkv = None                            # the position part did the projection too
        else:
            qkv = ops.linear(h, self.w_qkv, out_dtype=torch.float32)
        if qkv is None:
            pass
        elif position is not None and hasattr(position, "apply_and_store"):
            # the position part does it all: q/k norm, its own encoding, queries out, keys and values stored
            position.apply_and_store(qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, ctx, cache, q,
                                     self.H, self.K, self.hd)
        else:
            ops.qk_norm_rope_store(qkv, self.q_norm_w, self.k_norm_w,
                                   position.table() if position is not None else None, ctx.positions,
                                   cache.slots, q, cache.k, cache.v, self.H, self.K, self.hd,
                                   cache.block_size, self.qk_norm_eps, write_kv=cache.write)
        attn = torch.empty_like(q)
        ops.paged_attention(q, cache.k, cache.v, attn, ctx, cache.block_table, self.H, self.K, self.hd,
                            cache.block_size, self.scale, self.window)
        if residual is not None:
            if then_norm is not None:
                return ops.linear(attn, self.w_o, out=residual, accumulate=True, then_norm=then_norm)
            ops.linear(attn, self.w_o, out=residual, accumulate=True)
            return None
        return ops.linear(attn, self.w_o, out_dtype=torch.float32)
