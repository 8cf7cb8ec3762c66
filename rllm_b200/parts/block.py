"""How a layer's parts are arranged.  ``pre_norm``:

    x += pending;  a = mixer(norm_mixer(x));  x += a;  f = ffn(norm_ffn(x));  pending = f

A mixer or feed-forward is handed the float32 residual stream as `residual`; it may add its
output into it itself (its last product accumulates into x) and return None, or ignore it and
return its output, which the next norm then adds in the same kernel that normalizes
(AxiomOperator/rllm fuses the next layer's norm into the residual add:
crates/rllm-model/src/qwen3.rs:192-208).

A block's interface: ``__init__(layer_spec, runtime)`` builds its parts from the registries;
``parts()`` lists them; ``forward(x, pending, ctx, cache) -> pending``.
"""
from __future__ import annotations

from .base import build_part, register_part


@register_part("block", "pre_norm")
class PreNormBlock:
    def __init__(self, layer_spec, runtime):
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], runtime)
        self.norm_ffn = build_part("norm", layer_spec.norms["ffn"], runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime)
        self.ffn = build_part("ffn", layer_spec.ffn, runtime)
        self.position = (build_part("position", layer_spec.position, runtime)
                         if layer_spec.position is not None else None)

    def parts(self):
        ps = [self.norm_mixer, self.mixer, self.norm_ffn, self.ffn]
        if self.position is not None:
            ps.append(self.position)
        return ps

    def forward(self, x, pending, ctx, cache):
        h = self.norm_mixer.forward(x, pending)
        a = self.mixer.forward(h, ctx, cache, self.position, residual=x)
        h = self.norm_ffn.forward(x, a)
        return self.ffn.forward(h, ctx, residual=x)
