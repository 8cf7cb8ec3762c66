"""The step function: runs one flat batch of (request, its next tokens) from the cache and
returns the logits at the wanted places.

`Engine.step(items)` appends every item's tokens to its request (all-or-nothing: if the pages
do not suffice nothing has changed), uploads the step's index arrays in one copy, runs the
model over exactly the given tokens and returns float32 logits ``[wanted, vocab]`` on the
device, in the order of the items and of their `want`.  Pages that a window has passed are
given back after the step; `finish(request)` gives back everything a request holds.

AxiomOperator/rllm: ``KvPool::step_sampled`` (crates/rllm-model/src/generate.rs:85-139) with
the same pre-checks before any mutation (86-100).
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages, PagedKVView, StateView
from .batch import StepContext, StepItem


class StepError(ValueError):
    """A step that cannot run as given (empty item, bad token id, bad `want`, unknown request)."""


class Engine:
    def __init__(self, model, block_size: int = 16, max_tokens: int = 4096, max_requests: int = 64):
        if not model.loaded:
            raise ValueError("the model has no weights loaded")
        self.model = model
        self.runtime = model.runtime
        if self.runtime.device.type != "cuda":
            raise RuntimeError("rllm_b200 runs on a CUDA device only; there is no CPU path "
                               f"(got device {self.runtime.device})")
        self.vocab_size = model.spec.vocab_size
        needs, cache_of = model.cache_needs()
        self.cache = CacheManager(needs, cache_of, block_size, max_tokens, max_requests)
        self.cache.allocate_device(self.runtime.device, self.runtime.dtype)
        self.block_size = block_size
        self._staging = []
        self._staging_events = []
        self._staging_next = 0
        self.stats = {"steps": 0, "step_tokens": 0}
        self.last_upload_bytes = 0

    # ------------------------------------------------------------------ staging
    def _upload(self, arrays: Sequence[np.ndarray]):
        """Copies int32 arrays to the device through one pinned buffer; returns device views.
        Each array starts on a 16-byte boundary."""
        offs, total = [], 0
        for a in arrays:
            offs.append(total)
            total += (a.size + 3) // 4 * 4
        total = max(total, 4)
        if not self._staging or self._staging[0].numel() < total:
            cap = max(4096, 1 << (total - 1).bit_length())
            for ev in self._staging_events:
                ev.synchronize()
            self._staging = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._staging_events = [torch.cuda.Event() for _ in range(4)]
        i = self._staging_next
        self._staging_next = (i + 1) % len(self._staging)
        self._staging_events[i].synchronize()
        host = self._staging[i]
        hv = host.numpy()
        for a, o in zip(arrays, offs):
            hv[o:o + a.size] = a.reshape(-1)
        dev = torch.empty(total, dtype=torch.int32, device=self.runtime.device)
        dev.copy_(host[:total], non_blocking=True)
        self.last_upload_bytes = 4 * total
        self._staging_events[i].record()
        return [dev[o:o + a.size].view(a.shape) for a, o in zip(arrays, offs)]

    # ------------------------------------------------------------------ the step
    def step(self, items: Sequence[StepItem]) -> Optional[torch.Tensor]:
        ctx, views = self.prepare(items)
        logits = self.model.forward(ctx, views)
        self.after_step(items)
        return logits

    def prepare(self, items: Sequence[StepItem]):
        """Validates, appends to the cache and builds the step's context and cache views."""
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
            for t in it.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise StepError(f"request {it.request_id!r}: token id {t} is outside the "
                                    f"vocabulary of {self.vocab_size}")
            for w in it.want:
                if not 0 <= int(w) < k:
                    raise StepError(f"request {it.request_id!r}: wanted place {w} is outside its "
                                    f"{k} tokens")
        cache = self.cache
        cache.check_append([(it.request_id, len(it.tokens)) for it in items])   # raises OutOfPages

        n = sum(len(it.tokens) for it in items)
        R = len(items)
        tokens = np.empty(n, np.int32)
        positions = np.empty(n, np.int32)
        seq_ids = np.empty(n, np.int32)
        cu_q = np.zeros(R + 1, np.int32)
        ctx_lens = np.empty(R, np.int32)
        state_slots = np.empty(R, np.int32)
        rows = []
        group_slots = [np.empty(n, np.int32) for _ in cache.paged]
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
        tables = []
        for g in range(len(cache.paged)):
            tl = [cache.block_table(it.request_id, g) for it in items]
            width = max(1, max(len(t) for t in tl))
            tab = np.zeros((R, width), np.int32)
            for r, t in enumerate(tl):
                tab[r, :len(t)] = t
            tables.append(tab)
        logit_rows = np.asarray(rows, np.int32)
        arrays = [tokens, positions, seq_ids, cu_q, ctx_lens, state_slots, logit_rows, *group_slots, *tables]
        dev = self._upload(arrays)
        G = len(cache.paged)
        ctx = StepContext(
            n_tokens=n, n_requests=R, tokens=dev[0], positions=dev[1], seq_ids=dev[2], cu_q=dev[3],
            ctx_lens=dev[4], state_slots=dev[5], logit_rows=dev[6] if len(rows) else None,
            q_lens=q_lens, start_pos=start_pos, ctx_lens_host=[int(c) for c in ctx_lens],
            max_q_len=max(q_lens), max_ctx_len=int(ctx_lens.max()))
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
        self.stats["steps"] += 1
        self.stats["step_tokens"] += n
        return ctx, views

    def after_step(self, items: Sequence[StepItem]) -> None:
        for it in items:
            self.cache.release_passed(it.request_id)

    def finish(self, request_id) -> None:
        """Gives back what a finished request holds.  Freed pages may be handed out again at once:
        kernels of earlier steps that read them are ordered before later writes by the stream."""
        if self.cache.has(request_id):
            self.cache.free(request_id)
