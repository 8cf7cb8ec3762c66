"""What every part of a layer has in common, the registries of part kinds, and what a
mixer may ask of the cache manager.

A part is built from a :class:`~rllm_b200.config.base.PartSpec` (its kind, its sizes and
constants, the prefix of its tensors) and a :class:`Runtime`.  It says which tensors it
expects (`expected_tensors`), takes them (`load`), and is then called by its block.  No part
knows which model it is in.  A new kind is added with ``@register_part(category, kind)``:
nothing else in the package has to change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional

import torch

CATEGORIES = ("embedding", "norm", "position", "mixer", "ffn", "block", "lm_head")
_REGISTRY: dict[str, dict[str, Callable]] = {c: {} for c in CATEGORIES}


class PartError(ValueError):
    pass


def register_part(category: str, kind: str):
    """Class decorator: makes `kind` available in `category` ('mixer', 'ffn', 'norm', ...)."""
    if category not in _REGISTRY:
        raise PartError(f"unknown part category {category!r} (known: {', '.join(CATEGORIES)})")

    def deco(cls):
        _REGISTRY[category][kind] = cls
        return cls
    return deco


def part_class(category: str, kind: str):
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise PartError(f"no {category} part of kind {kind!r} is registered "
                        f"(registered: {', '.join(sorted(_REGISTRY.get(category, {})))})") from None


def build_part(category: str, spec, runtime: "Runtime", **extra):
    return part_class(category, spec.kind)(dict(spec.params), spec.prefix, runtime, **extra)


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision a model runs.  `dtype` is the storage type of weights,
    activations between kernels and the cache (bfloat16 or float32); the residual stream,
    norms' statistics, softmax, rotation angles and logits are float32 in both."""
    device: torch.device
    dtype: torch.dtype

    @property
    def is_f32(self) -> bool:
        return self.dtype == torch.float32


# ---------------------------------------------------------------- what a mixer asks of the cache

@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values in pages.  `window` > 0: only the last `window` keys are ever read, so
    pages that the window has passed can be given back."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request (any shape), kept in a slot for the request's lifetime
    and zeroed when the slot is taken."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts."""

    # True for a part whose `forward` may be captured into a CUDA graph and replayed for another step
    # of the same padded shape: it launches kernels and torch operations on device tensors only, reads
    # nothing back to the host, and takes from the step's host copies (`ctx.q_lens`, `ctx.start_pos`,
    # ...) no more than the shape.  Padding rows of such a step have slot -1 in the pages and the last
    # state slot, which belongs to no request.  A model with a part that does not say so runs eagerly.
    CAPTURE_SAFE = False

    # True for a part that touches device memory through the launchers of csrc/ops only (no torch
    # operation of its own on tensors): the launches of a layer of such parts can be recorded once and
    # replayed for the other layers of the same build (models/model.py, ops.Trace).
    TRACEABLE = False

    def __init__(self, params: Mapping[str, Any], prefix: str, runtime: Runtime):
        self.params = dict(params)
        self.prefix = prefix
        self.runtime = runtime

    def expected_tensors(self) -> dict:
        """Full tensor name -> (shape, role); role 'norm' marks weights that start at 1."""
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Takes the tensors named by `expected_tensors` (CPU, as stored) and keeps device copies."""

    def _to_device(self, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return t.to(device=self.runtime.device, dtype=dtype or self.runtime.dtype).contiguous()


class Mixer(Part):
    """Token mixer interface.

    ``cache_need()`` returns a PagedKVNeed, a StateNeed or None.
    ``forward(h, ctx, cache, position)``: `h` [n, hidden] normed activations in the runtime's
    dtype, `ctx` the step's :class:`~rllm_b200.engine.batch.StepContext`, `cache` the view of
    this run entry's cache (:class:`~rllm_b200.cache.views.PagedKVView` or ``StateView``; None
    if it needs none), `position` the layer's position-encoding part or None, `residual` the
    float32 residual stream [n, hidden].  Returns the mixer's output [n, hidden] (float32 or the
    runtime's dtype), which the block adds to the residual stream; or adds it into `residual`
    itself and returns None."""

    def cache_need(self):
        return None

    def forward(self, h, ctx, cache, position, residual=None):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(h, ctx, residual=None)`` -> [n, hidden] or None.  As for mixers, a part may add
    its output into the float32 `residual` itself and return None."""

    def forward(self, h, ctx, residual=None):
        raise NotImplementedError


class Norm(Part):
    """``forward(x, delta=None, rows=None, write_x=True)``: adds `delta` to the float32 residual
    stream `x` (in place when write_x), optionally gathers `rows`, returns the normed rows in the
    runtime's dtype."""

    def forward(self, x, delta=None, rows=None, write_x=True):
        raise NotImplementedError
