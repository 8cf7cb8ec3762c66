"""How a layer's parts are arranged.  ``pre_norm``:

    x += pending;  a = mixer(norm_mixer(x));  x += a;  f = ffn(norm_ffn(x));  pending = f

A mixer or feed-forward is handed the float32 residual stream as `residual`; it may add its
output into it itself (its last product accumulates into x) and return None, or ignore it and
return its output, which the next norm then adds in the same kernel that normalizes
(AxiomOperator/rllm fuses the next layer's norm into the residual add:
crates/rllm-model/src/qwen3.rs:192-208).

A block's interface: ``__init__(layer_spec, runtime)`` builds its parts from the registries;
``parts()`` lists them; ``forward(x, pending, ctx, cache) -> pending``.

Optional, for blocks that set ``DEFERS_NORM``: ``entry()`` returns the block's first norm and the
part behind it, and ``forward`` takes ``next_entry`` (the same pair of the block that runs next).
A norm that stands between two weight-streaming products of a decode step then needs no kernel of
its own: the product before it prepares it (``then_norm``) and hands the rows on as
``ops.NormedRows``, which the product after it divides by the rms.  ``pending`` is then that
object: the residual stream is complete and the next block's first norm is under way.  Whether
this happens is decided per step from the parts on both sides (``first_product`` / ``last_product``,
``deferrable``) and the number of rows; parts or norms without these methods get the plain path.
"""
from __future__ import annotations

from ..csrc import ops
from .base import build_part, register_part


def deferral(before, norm, after, m: int):
    """(weight, eps) if `norm`, between the parts `before` and `after`, can be deferred at m rows."""
    last, first, able = (getattr(before, "last_product", None), getattr(after, "first_product", None),
                         getattr(norm, "deferrable", None))
    if last is None or first is None or able is None or before.runtime.is_f32:
        return None
    w_before, w_lead, swiglu_lead = last()
    w_after, swiglu_after = first()
    if not ops.defers_norm(m, w_before, w_after, swiglu_after, w_lead, swiglu_lead):
        return None
    return able()


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

    DEFERS_NORM = True
    CAPTURE_SAFE = True
    TRACEABLE = True

    def entry(self):
        return self.norm_mixer, self.mixer

    def forward(self, x, pending, ctx, cache, next_entry=None):
        m = x.shape[0]
        h = pending if isinstance(pending, ops.NormedRows) else self.norm_mixer.forward(x, pending)
        later = deferral(self.mixer, self.norm_ffn, self.ffn, m)
        if later is not None:
            h = self.mixer.forward(h, ctx, cache, self.position, residual=x, then_norm=later)
        else:
            a = self.mixer.forward(h, ctx, cache, self.position, residual=x)
            h = self.norm_ffn.forward(x, a)
        later = deferral(self.ffn, next_entry[0], next_entry[1], m) if next_entry is not None else None
        if later is not None:
            return self.ffn.forward(h, ctx, residual=x, then_norm=later)
        return self.ffn.forward(h, ctx, residual=x)
