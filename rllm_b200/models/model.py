"""A decoder put together from a :class:`~rllm_b200.config.base.ModelSpec`: embedding, layers
(blocks of parts), final norm, LM head, and the run order as data.  This file knows no
architecture; AxiomOperator/rllm's counterpart is the layer loop of
crates/rllm-model/src/qwen3.rs:162-234, written once per architecture there.
"""
from __future__ import annotations

import os
from pathlib import Path

import torch

from ..config import ModelConfig, ModelSpec, load_config
from ..parts import Runtime, build_part, part_class
from ..weights.loader import load_checked


TRACE_LAYERS = os.environ.get("RLLM_B200_NO_LAYER_TRACE", "0") in ("", "0")


def _tensors_of(obj) -> dict:
    """attribute name -> device tensor of an object (a part's weights, a cache view's planes)."""
    return {k: v for k, v in vars(obj).items() if isinstance(v, torch.Tensor) and v.is_cuda}


class _LayerTrace:
    """The launches of one run entry, recorded, with what a replay for another entry of the same
    build has to swap: the tensors of the block's parts, of the entry's cache view, of the norm
    that follows the block (a product may prepare it), and the rows that came in."""

    def __init__(self, trace, block, view, nxt, pending_in, pending_out):
        self.trace, self.pending_out = trace, pending_out
        self.fixed = self._fixed_roles(block, nxt)            # [address, ...] in a fixed order
        self.view = self._view_roles(view)
        self.inputs = self._pending_pointers(pending_in)
        trace.freeze(self.fixed + self.view + self.inputs)

    @staticmethod
    def _fixed_roles(block, nxt) -> list:
        """Addresses of the tensors of the block's parts and of the norm behind it; they never change,
        so they are worked out once per (block, follower)."""
        cache = block.__dict__.setdefault("_role_addresses", {})
        key = id(nxt)
        out = cache.get(key)
        if out is None:
            out = []
            for part in block.parts() + ([nxt.entry()[0]] if nxt is not None else []):
                out += [t.data_ptr() for _, t in sorted(_tensors_of(part).items())]
            cache[key] = out
        return out

    @staticmethod
    def _view_roles(view) -> list:
        if view is None:
            return []
        return [t.data_ptr() for _, t in sorted(_tensors_of(view).items())]

    @staticmethod
    def _pending_pointers(pending) -> list:
        from ..csrc import ops
        if isinstance(pending, ops.NormedRows):
            return [pending.xw.data_ptr(), pending.ssq.data_ptr()]
        if isinstance(pending, torch.Tensor):
            return [pending.data_ptr()]
        return []

    def replay(self, block, view, nxt, pending_in):
        self.trace.replay(self._fixed_roles(block, nxt) + self._view_roles(view) + self._pending_pointers(pending_in))
        return self.pending_out


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.runtime = spec, runtime
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = [part_class("block", ls.block)(ls, runtime) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.lm_head = build_part("lm_head", spec.lm_head, runtime)
        self.run_order = list(spec.run_order)
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"run entry {i} names layer {e.layer}, but there are {len(self.blocks)}")
        self.loaded = False
        # decode steps of this model may be captured into CUDA graphs: every part says it can be
        self.capture_safe = all(getattr(p, "CAPTURE_SAFE", False) for p in self._weighted_parts() + self.blocks)
        # The layers of a step that launches from Python are traced once per build and replayed for the
        # other layers of that build (ops.Trace).  A block's build: its class, its parts' kinds and
        # parameters; only blocks all of whose parts launch through ops alone (TRACEABLE) take part.
        self._builds = [self._build_key(b) for b in self.blocks]

    @staticmethod
    def _build_key(block):
        if not getattr(block, "TRACEABLE", False) or not hasattr(block, "entry"):
            return None
        parts = block.parts()
        if not all(getattr(p, "TRACEABLE", False) for p in parts):
            return None
        return (type(block).__name__,) + tuple((type(p).__name__, repr(sorted(p.params.items()))) for p in parts)

    # ------------------------------------------------------------------ tensors
    def _weighted_parts(self):
        ps = [self.embedding]
        for b in self.blocks:
            ps.extend(b.parts())
        ps += [self.final_norm, self.lm_head]
        return ps

    def expected_tensors(self) -> dict:
        out = {}
        for p in self._weighted_parts():
            out.update(p.expected_tensors())
        return out

    def ignorable_tensors(self) -> set:
        out = set()
        for p in self._weighted_parts():
            if hasattr(p, "ignorable_tensors"):
                out |= p.ignorable_tensors()
        return out

    def load_tensors(self, tensors: dict) -> None:
        """`tensors`: name -> tensor (CPU or device), already checked against expected_tensors()."""
        shared = {}
        for p in self._weighted_parts():
            if p is self.lm_head:
                continue
            p.load(tensors)
        shared[self.embedding.prefix + "weight"] = self.embedding.weight
        self.lm_head.load(tensors, shared=shared)
        self.loaded = True

    def load_dir(self, model_dir) -> None:
        exp = {n: shape for n, (shape, _) in self.expected_tensors().items()}
        self.load_tensors(load_checked(model_dir, exp, self.ignorable_tensors()))

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self):
        """(needs, cache_of) per run entry, for the cache manager."""
        needs = [self.blocks[e.layer].mixer.cache_need() for e in self.run_order]
        return needs, [e.cache_of for e in self.run_order]

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, views):
        """Runs the step's tokens through the run order; returns float32 logits [wanted, vocab]
        (None when no row is wanted).  `views[i]` is run entry i's cache view."""
        ctx.scratch = {}                 # what the layers of this pass share (a captured pass makes its own again)
        x = self.embedding.forward(ctx.tokens)
        pending = None
        from ..csrc import ops
        traces = {} if (TRACE_LAYERS and x.is_cuda and ops.can_trace()) else None
        for i, e in enumerate(self.run_order):
            block = self.blocks[e.layer]
            nxt = self.blocks[self.run_order[i + 1].layer] if i + 1 < len(self.run_order) else None
            defers = getattr(block, "DEFERS_NORM", False) and getattr(nxt, "DEFERS_NORM", False)
            key = None
            if traces is not None and self._builds[e.layer] is not None:
                view = views[i]
                # entries replay one another when they are built alike, read and write caches of the same
                # kind through the same table, got rows of the same kind and are followed alike
                key = (self._builds[e.layer], type(view).__name__, getattr(view, "group", None),
                       getattr(view, "write", None), type(pending).__name__,
                       self._builds[self.run_order[i + 1].layer] if defers else None)
                rec = traces.get(key)
                if rec is not None:
                    pending = rec.replay(block, view, nxt if defers else None, pending)
                    continue
            if key is not None:
                with ops.tracing() as trace:
                    out = (block.forward(x, pending, ctx, views[i], next_entry=nxt.entry()) if defers
                           else block.forward(x, pending, ctx, views[i]))
                traces[key] = _LayerTrace(trace, block, views[i], nxt if defers else None, pending, out)
                pending = out
            elif defers:
                pending = block.forward(x, pending, ctx, views[i], next_entry=nxt.entry())
            else:
                pending = block.forward(x, pending, ctx, views[i])
        if ctx.logit_rows is None or ctx.logit_rows.numel() == 0:
            return None
        h = self.final_norm.forward(x, pending, rows=ctx.logit_rows, write_x=False)
        return self.lm_head.forward(h)


def expected_tensors(spec: ModelSpec) -> dict:
    """name -> (shape, role) of every tensor a model of `spec` reads (no device needed)."""
    return DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32)).expected_tensors()


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
    elif str(dtype).lower() in ("bfloat16", "bf16"):
        return torch.bfloat16
    elif str(dtype).lower() in ("float32", "fp32", "f32"):
        return torch.float32
    raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")


def load_model(model_dir, dtype="bfloat16", device="cuda:0"):
    """config.json chooses the model class (through the architecture registry); weights come from
    model.safetensors.  Returns (config, DecoderModel)."""
    config = load_config(model_dir)
    model = DecoderModel(config.model_spec(), Runtime(torch.device(device), parse_dtype(dtype)))
    model.load_dir(Path(model_dir))
    return config, model


def random_model(config: ModelConfig, seed=0, dtype="bfloat16", device="cuda:0", std=0.02, norm_std=0.1,
                 generate_on_device=False):
    """A model with random weights without going through a file (large benchmarks)."""
    from ..weights.random_init import random_tensors
    rt = Runtime(torch.device(device), parse_dtype(dtype))
    model = DecoderModel(config.model_spec(), rt)
    tensors = random_tensors(model.expected_tensors(), seed, rt.dtype, std, norm_std,
                             device=device if generate_on_device else "cpu")
    model.load_tensors(tensors)
    return model
