"""The step function: runs one flat batch of (request, its next tokens) from the cache and
returns the logits at the wanted places.

`Engine.step(items)` appends every item's tokens to its request (all-or-nothing: if the pages
do not suffice nothing has changed), uploads the step's index arrays in one copy, runs the
model over exactly the given tokens and returns float32 logits ``[wanted, vocab]`` on the
device, in the order of the items and of their `want`.  Pages that a window has passed are
given back after the step; `finish(request)` gives back everything a request holds.

Steps that hold one token per request (decode) are replayed from CUDA graphs: one graph per
(padded number of requests, padded context length), captured the second time a shape is seen,
with the step's index arrays copied into the graph's fixed input buffer before each replay.
So are steps of one-token items followed by ONE portion of a prompt (what the scheduler makes of
decoding requests beside the short tail of a prompt, and a lone short portion too; up to
GRAPH_MAX_PORTION tokens): the shape then also holds the portion's length.  Other steps launch
their kernels one by one from Python, about 17 us of host time each.

AxiomOperator/rllm: ``KvPool::step_sampled`` (crates/rllm-model/src/generate.rs:85-139) with
the same pre-checks before any mutation (86-100); graph replay keyed by the step's shape
(crates/rllm-model/src/lib.rs:78-95, crates/rllm-cuda/src/backend.rs:1394-1430).
"""
from __future__ import annotations

import contextlib
import math
import os
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, PagedKVView, StateView
from ..cache.native import NativeCacheManager
from ..csrc import ops, profiler
from .batch import StepContext, StepItem


class StepError(ValueError):
    """A step that cannot run as given (empty item, bad token id, bad `want`, unknown request)."""


GRAPH_MAX_REQUESTS = 64
GRAPH_CTX_QUANTUM = 256          # context lengths are padded to a multiple of this many tokens
GRAPH_CACHE_MAX = 48             # captured shapes kept per engine
GRAPH_PORTION_CAPTURE_AT = 4     # a shape with a prompt portion is captured when it comes for this many-th time
# Longest prompt portion of a step that is replayed from a graph (0: only decode steps are).  The
# reference replays steps of up to 8 tokens (crates/rllm-model/src/lib.rs:80-87).  Longer portions
# work the same way (the tests run them), but do not pay: their shapes repeat seldom, and padding the
# decoding requests beside them to a power of two can push the products over a tile boundary (measured
# on the 8B serving workload with portions of 512: 4.7 % slower than launching those steps one by one).
GRAPH_MAX_PORTION = int(os.environ.get("RLLM_B200_GRAPH_MAX_PORTION", "8"))


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class _Layout:
    """Where each int32 array of a step lies in the flat upload buffer (16-byte aligned starts)."""

    def __init__(self, shapes: Sequence[tuple]):
        self.shapes, self.offsets, total = list(shapes), [], 0
        for shp in self.shapes:
            self.offsets.append(total)
            total += (math.prod(shp) + 3) // 4 * 4
        self.total = max(total, 4)

    def views(self, flat: torch.Tensor):
        return [flat[o:o + math.prod(s)].view(s) for s, o in zip(self.shapes, self.offsets)]


class _DecodeGraph:
    def __init__(self):
        self.uses = 0
        self.static = None       # device int32 buffer the graph reads
        self.layout = None
        self.ctx = None
        self.views = None
        self.graph = None
        self.logits = None
        self.launches = 0
        self.last_used = 0


class Engine:
    def __init__(self, model, block_size: int = 32, max_tokens: int = 4096, max_requests: int = 64,
                 use_graphs: bool = True, native_host: bool = True, max_step_tokens: Optional[int] = None):
        """`native_host`: page accounting and the step's index arrays are built by the C++ host
        runtime (default); False keeps them in Python (same results, slower).  `max_step_tokens`: a
        promise that no step brings more tokens of one request than this (a scheduler's portion size);
        layers that read a window of keys then share a smaller pool of pages (see CacheManager)."""
        if not model.loaded:
            raise ValueError("the model has no weights loaded")
        self.model = model
        self.runtime = model.runtime
        if self.runtime.device.type != "cuda":
            raise RuntimeError("rllm_b200 runs on a CUDA device only; there is no CPU path "
                               f"(got device {self.runtime.device})")
        self.vocab_size = model.spec.vocab_size
        needs, cache_of = model.cache_needs()
        self.native_host = native_host
        manager = NativeCacheManager if native_host else CacheManager
        self.cache = manager(needs, cache_of, block_size, max_tokens, max_requests, max_step_tokens)
        self.cache.allocate_device(self.runtime.device, self.runtime.dtype)
        # a request never grows beyond the positions the model has: the append that would take it
        # there is refused before anything changes (RequestTooLong)
        self.cache.set_max_length(int(getattr(model.spec, "max_position", 0) or 0))
        self.block_size = block_size
        self._windowed = any(g.need.window > 0 for g in self.cache.paged)     # only then do pages fall out of reach
        # RLLM_B200_NO_GRAPHS=1 turns graph replay off (the reference's RLLM_NO_GRAPHS); the profiling
        # switch does too: events cannot be recorded into a capture
        # and a model one of whose parts does not declare itself safe to capture (CAPTURE_SAFE) runs eagerly
        self.use_graphs = (use_graphs and not profiler.enabled() and getattr(model, "capture_safe", False)
                           and os.environ.get("RLLM_B200_NO_GRAPHS", "0") in ("", "0"))
        self._graphs: dict = {}
        self._graph_pool = None
        self._staging = []
        self._staging_events = []
        self._staging_next = 0
        self.stats = {"steps": 0, "step_tokens": 0, "graph_replays": 0, "graphs_captured": 0}
        self.last_upload_bytes = 0

    # ------------------------------------------------------------------ staging
    def _staging_buffer(self, total: int) -> torch.Tensor:
        """The next pinned buffer of a ring of four (each reused only after its last copy has
        finished), at least `total` int32 long."""
        if not self._staging or self._staging[0].numel() < total:
            cap = max(4096, 1 << (total - 1).bit_length())
            for ev in self._staging_events:
                ev.synchronize()
            self._staging = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._staging_events = [torch.cuda.Event() for _ in range(4)]
        i = self._staging_next
        self._staging_next = (i + 1) % len(self._staging)
        self._staging_events[i].synchronize()
        self._staged = i
        return self._staging[i]

    def _stage(self, arrays: Sequence[np.ndarray], layout: _Layout) -> torch.Tensor:
        """Packs the arrays into a pinned buffer and returns the pinned slice to copy from."""
        total = layout.total
        buf = self._staging_buffer(total)
        hv = buf.numpy()
        for a, o in zip(arrays, layout.offsets):
            hv[o:o + a.size] = a.reshape(-1)
        self.last_upload_bytes = 4 * total
        return buf[:total]

    def _build(self, items: Sequence[StepItem], pad_requests: int = 0, pad_width: int = 0):
        """Appends the items to the cache and stages the step's arrays in pinned memory.
        Returns (pinned slice, layout, meta)."""
        if not self.native_host:
            arrays, meta = self._arrays(items, pad_requests, pad_width)
            layout = _Layout([a.shape for a in arrays])
            return self._stage(arrays, layout), layout, meta
        return self._finish_build(items, pad_requests, *self._build_native(items, pad_requests, pad_width))

    def _finish_build(self, items, pad_requests: int, buf, offsets, m):
        """Layout and host-side shape of a step that the C++ builder has written into `buf`."""
        n, R, n_rows, width, total = m[:5]
        G = len(self.cache.paged)
        shapes = [(n,), (n,), (n,), (R + 1,), (R,), (R,), (n_rows,)] + [(n,)] * G + [(R, width)] * G
        layout = _Layout(shapes)
        assert layout.offsets == offsets and layout.total == total
        hv = buf.numpy()
        cu = hv[offsets[3]:offsets[3] + R + 1]
        q_lens = np.diff(cu).tolist()
        start_pos = hv[offsets[1] + cu[:-1]].tolist()
        ctx_lens = hv[offsets[4]:offsets[4] + R].tolist()
        rows = hv[offsets[6]:offsets[6] + n_rows].tolist() if not pad_requests else \
            [int(cu[i]) + int(w) for i, it in enumerate(items) for w in it.want]
        meta = dict(n=n, R=R, q_lens=q_lens, start_pos=start_pos, rows=rows, ctx_lens=ctx_lens)
        self.last_upload_bytes = 4 * total
        return buf[:total], layout, meta

    def _build_native(self, items, pad_requests: int, pad_width: int, pad_quantum: int = 0):
        """The C++ step builder on the next pinned buffer: (buffer, offsets, (n, R, rows, width, total, longest))."""
        guess = 4096
        while True:
            buf = self._staging_buffer(guess)
            offsets, m, _ = self.cache.build_step(items, self.vocab_size, buf, pad_requests, pad_width, pad_quantum)
            if offsets is not None:
                self.last_upload_bytes = 4 * m[4]
                return buf, offsets, m
            self._staging_next = self._staged            # the buffer was not used: hand it out again
            guess = m[4]

    def _copy_in(self, dev: torch.Tensor, host: torch.Tensor) -> None:
        dev.copy_(host, non_blocking=True)
        self._staging_events[self._staged].record()

    # ------------------------------------------------------------------ validation + cache append
    def _check_items(self, items: Sequence[StepItem]) -> None:
        if not items:
            raise StepError("a step needs at least one item")
        seen = set()
        for it in items:
            if it.request_id in seen:
                raise StepError(f"request {it.request_id!r} appears twice in one step")
            seen.add(it.request_id)
            k = len(it.tokens)
            if k == 0:
                raise StepError(f"request {it.request_id!r}: an item needs at least one token")
            toks = np.asarray(it.tokens)
            if toks.dtype.kind not in "iu" or toks.min() < 0 or toks.max() >= self.vocab_size:
                bad = next((t for t in it.tokens if not (isinstance(t, (int, np.integer)) and 0 <= t < self.vocab_size)), None)
                raise StepError(f"request {it.request_id!r}: token id {bad} is outside the "
                                f"vocabulary of {self.vocab_size}")
            for w in it.want:
                if not 0 <= int(w) < k:
                    raise StepError(f"request {it.request_id!r}: wanted place {w} is outside its "
                                    f"{k} tokens")
        self.cache.check_append([(it.request_id, len(it.tokens)) for it in items])   # raises OutOfPages

    def _arrays(self, items: Sequence[StepItem], pad_requests: int = 0, pad_width: int = 0):
        """Appends to the cache and builds the step's int32 arrays.  With `pad_requests`, the
        arrays are padded to that many one-token requests (padding rows write nothing: slot -1)
        and block tables to `pad_width` columns."""
        cache = self.cache
        R_real = len(items)
        n_real = sum(len(it.tokens) for it in items)
        R = max(R_real, pad_requests)
        n = n_real + (R - R_real)
        tokens = np.zeros(n, np.int32)
        positions = np.zeros(n, np.int32)
        seq_ids = np.arange(n, dtype=np.int32) if pad_requests else np.zeros(n, np.int32)
        cu_q = np.zeros(R + 1, np.int32)
        ctx_lens = np.ones(R, np.int32)
        state_slots = np.zeros(R, np.int32)
        rows = []
        group_slots = [np.full(n, -1, np.int32) for _ in cache.paged]
        q_lens, start_pos = [], []
        base = 0
        for r, it in enumerate(items):
            k = len(it.tokens)
            start = cache.length(it.request_id) if cache.has(it.request_id) else 0
            slots = cache.append(it.request_id, k)
            tokens[base:base + k] = it.tokens
            positions[base:base + k] = np.arange(start, start + k, dtype=np.int32)
            seq_ids[base:base + k] = r
            for g, s in enumerate(slots):
                group_slots[g][base:base + k] = s
            rows.extend(base + int(w) for w in it.want)
            cu_q[r + 1] = base + k
            ctx_lens[r] = start + k
            state_slots[r] = cache.state_slot(it.request_id)
            q_lens.append(k)
            start_pos.append(start)
            base += k
        for r in range(R_real, R):
            cu_q[r + 1] = cu_q[r] + 1
            state_slots[r] = cache.max_requests          # the state slot that belongs to no request
            q_lens.append(1)
            start_pos.append(0)
        tables = []
        for g in range(len(cache.paged)):
            tl = [cache.block_table(it.request_id, g) for it in items]
            width = max(1, pad_width, max(len(t) for t in tl))
            tab = np.zeros((R, width), np.int32)
            for r, t in enumerate(tl):
                tab[r, :len(t)] = t
            tables.append(tab)
        logit_rows = np.arange(n, dtype=np.int32) if pad_requests else np.asarray(rows, np.int32)
        arrays = [tokens, positions, seq_ids, cu_q, ctx_lens, state_slots, logit_rows, *group_slots, *tables]
        meta = dict(n=n, R=R, q_lens=q_lens, start_pos=start_pos, rows=rows,
                    ctx_lens=[int(c) for c in ctx_lens])
        return arrays, meta

    def _context(self, dev: Sequence[torch.Tensor], meta: dict, has_rows: bool):
        cache = self.cache
        G = len(cache.paged)
        ctx = StepContext(
            n_tokens=meta["n"], n_requests=meta["R"], tokens=dev[0], positions=dev[1], seq_ids=dev[2],
            cu_q=dev[3], ctx_lens=dev[4], state_slots=dev[5], logit_rows=dev[6] if has_rows else None,
            q_lens=meta["q_lens"], start_pos=meta["start_pos"], ctx_lens_host=meta["ctx_lens"],
            max_q_len=max(meta["q_lens"]), max_ctx_len=max(meta["ctx_lens"]))
        dev_slots, dev_tables = dev[7:7 + G], dev[7 + G:7 + 2 * G]
        views = []
        for i, place in enumerate(cache.entry_place):
            if place is None:
                views.append(None)
            elif place[0] == "kv":
                _, g, plane = place
                pool = cache.paged[g].pool
                views.append(PagedKVView(pool[plane, 0], pool[plane, 1], dev_tables[g], dev_slots[g],
                                         self.block_size, write=cache.cache_of[i] is None, group=g))
            else:
                _, g, plane = place
                views.append(StateView(cache.stateful[g].state[plane], ctx.state_slots,
                                       write=cache.cache_of[i] is None))
        return ctx, views

    # ------------------------------------------------------------------ the step
    def step(self, items: Sequence[StepItem], device_tokens: Optional[torch.Tensor] = None,
             n_device: Optional[int] = None) -> Optional[torch.Tensor]:
        """`device_tokens` (int32 on the device): the token ids of the first `n_device` items (all of
        them by default), which have one token each, are taken from there instead of from the items,
        whose `tokens` are then placeholders: ids that an earlier step's sampler left on the device go
        into the next step without a round trip over the host."""
        decode_only = bool(items) and all(len(it.tokens) == 1 for it in items)
        n_dev = 0
        if device_tokens is not None:
            n_dev = len(items) if n_device is None else int(n_device)
            if (not 0 <= n_dev <= len(items) or any(len(it.tokens) != 1 for it in items[:n_dev])
                    or device_tokens.numel() < n_dev or device_tokens.dtype != torch.int32):
                raise StepError("device_tokens needs one int32 id for each of the first n_device items, "
                                "which have one token each")
            if n_dev == 0:
                device_tokens = None
        # A decode-only step on the C++ host is checked there (token range, wanted places, a request
        # named twice, pages: all before anything changes); the Python check runs only to word the
        # error.  Anything that is not a plain int goes through the Python check first.
        light = self.native_host and decode_only and all(type(it.tokens[0]) is int for it in items)
        if not light:
            self._check_items(items)
        self.stats["steps"] += 1
        self.stats["step_tokens"] += sum(len(it.tokens) for it in items)
        graphable = self.use_graphs
        if graphable and decode_only and len(items) <= GRAPH_MAX_REQUESTS:
            try:
                logits = self._graph_step(items, device_tokens, n_dev=n_dev)
            except (ValueError, KeyError):
                if light:
                    self._check_items(items)         # raises the StepError that names the fault
                raise
        elif graphable and self.native_host and self._one_portion_last(items):
            logits = self._graph_step(items, device_tokens, portion=len(items[-1].tokens), n_dev=n_dev)
        else:
            host, layout, meta = self._build(items)
            dev = torch.empty(layout.total, dtype=torch.int32, device=self.runtime.device)
            self._copy_in(dev, host)
            if device_tokens is not None:
                dev[:n_dev].copy_(device_tokens[:n_dev])                    # the tokens are the first array, in item order
            ctx, views = self._context(layout.views(dev), meta, bool(meta["rows"]))
            logits = self.model.forward(ctx, views)
        if self._windowed:
            for it in items:
                self.cache.release_passed(it.request_id)
        return logits

    @staticmethod
    def _one_portion_last(items) -> bool:
        """One-token items (at most GRAPH_MAX_REQUESTS, possibly none) and then one portion of
        2 to GRAPH_MAX_PORTION tokens of which at most the last one's logits are wanted."""
        last = items[-1]
        k = len(last.tokens)
        return (1 < k <= GRAPH_MAX_PORTION and len(items) - 1 <= GRAPH_MAX_REQUESTS
                and all(len(it.tokens) == 1 for it in items[:-1])
                and all(int(w) == k - 1 for w in last.want) and len(last.want) <= 1
                and all(len(it.want) <= 1 for it in items[:-1]))

    @contextlib.contextmanager
    def _capture(self, graph):
        """Stream capture into `graph` on a side stream, from the pool that all of this engine's
        graphs share (only one of them runs at a time, and a step's logits are valid until the next
        step).  Unlike torch.cuda.graph() it does not empty the caching allocator first: that
        costs most of a second each time a request grows into a new context bucket, and
        cudaMalloc calls for a while after."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph.capture_begin(pool=self._graph_pool)
            try:
                yield
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(side)

    def _graph_step(self, items: Sequence[StepItem], device_tokens=None, portion: int = 0, n_dev: int = 0) -> Optional[torch.Tensor]:
        """portion: 0 for a decode step; else the last item is a portion of that many tokens and the
        items before it have one token each (padded to a power of two, the portion behind them)."""
        R = len(items) - (1 if portion else 0)             # one-token items
        B = _bucket(R)
        if self.native_host:
            # the C++ builder finds the longest request and pads the tables itself: one call per step
            buf, offsets, m = self._build_native(items, B, 0, GRAPH_CTX_QUANTUM)
            ctx_pad = -(-m[5] // GRAPH_CTX_QUANTUM) * GRAPH_CTX_QUANTUM
            key = (B, portion, ctx_pad)
            g = self._graphs.get(key)
            if g is None:
                host, layout, meta = self._finish_build(items, B, buf, offsets, m)
            else:
                host, layout, meta = buf[:m[4]], None, None
                assert offsets == g.layout.offsets
        else:
            longest = max((self.cache.length(it.request_id) if self.cache.has(it.request_id) else 0) + 1
                          for it in items)
            ctx_pad = -(-longest // GRAPH_CTX_QUANTUM) * GRAPH_CTX_QUANTUM
            key = (B, 0, ctx_pad)
            host, layout, meta = self._build(items, pad_requests=B, pad_width=-(-ctx_pad // self.block_size))
            g = self._graphs.get(key)
        if g is None:
            if len(self._graphs) >= GRAPH_CACHE_MAX:
                # the least recently used shape goes (requests grow through context buckets and do not come back)
                del self._graphs[min(self._graphs, key=lambda k: self._graphs[k].last_used)]
            g = self._graphs[key] = _DecodeGraph()
            g.layout = layout
            g.static = torch.zeros(g.layout.total, dtype=torch.int32, device=self.runtime.device)
            # host-side shape of the step as the graph sees it: every request at the padded length
            if portion:
                meta_pad = dict(meta, start_pos=[ctx_pad - 1] * B + [ctx_pad - portion], ctx_lens=[ctx_pad] * (B + 1),
                                q_lens=[1] * B + [portion])
            else:
                meta_pad = dict(meta, start_pos=[ctx_pad - 1] * B, ctx_lens=[ctx_pad] * B, q_lens=[1] * B)
            g.ctx, g.views = self._context(g.layout.views(g.static), meta_pad, True)
        elif layout is not None:
            assert layout.offsets == g.layout.offsets
        self._copy_in(g.static, host)
        if device_tokens is not None:
            g.static[:n_dev].copy_(device_tokens[:n_dev])                  # the tokens are the first array, one-token items first
        g.uses += 1
        g.last_used = self.stats["steps"]
        if g.uses == 1 or (portion and g.uses < GRAPH_PORTION_CAPTURE_AT and g.graph is None):
            # first time: run the padded step eagerly (loads kernels, builds the dispatch plans).  Shapes
            # with a portion come in many more kinds than decode shapes, and most come once or twice: they
            # are captured (which costs more than running them) only when they have come a few times.
            g.logits = self.model.forward(g.ctx, g.views)
        else:
            if g.graph is None:
                before = ops.launch_count()
                graph = torch.cuda.CUDAGraph()
                with self._capture(graph):
                    g.logits = self.model.forward(g.ctx, g.views)
                g.graph, g.launches = graph, ops.launch_count() - before
                self.stats["graphs_captured"] += 1
            else:
                ops.add_launches(g.launches)
            g.graph.replay()
            self.stats["graph_replays"] += 1
        # the graph's logit rows: one per (padded) one-token item, then the portion's last row
        rows = [i for i, it in enumerate(items[:R]) for _ in it.want]
        if portion and items[-1].want:
            rows.append(B)
        if not rows:
            return None
        if rows == list(range(len(rows))) and (not portion or not items[-1].want):
            return g.logits[:len(rows)]
        return g.logits[torch.tensor(rows, dtype=torch.long, device=self.runtime.device)]

    def check_device_errors(self) -> None:
        """Raises if a kernel of an earlier step gave up a bounded wait (operand tiles that never
        arrived, a stage or accumulator that was never released): its results are then not to be
        used.  Reads one int from the device, so callers do it where they synchronize anyway."""
        ops.check_device_errors(self.runtime.device)

    def finish(self, request_id) -> None:
        """Gives back what a finished request holds.  Freed pages may be handed out again at once:
        kernels of earlier steps that read them are ordered before later writes by the stream."""
        if self.cache.has(request_id):
            self.cache.free(request_id)
