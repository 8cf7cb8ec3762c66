"""The cache manager: paged keys/values with a block table per request, one pool of pages per
group of layers with the same need, and slots for fixed-size per-request state.

Run entries (a layer at a place in the run order) that need the same thing (same number of
key/value heads, head size and window) form a *group*: they share one page allocator and one
block table per request, and each owns a plane of the group's device pool
``[entry, 2 (K,V), page, kv_head, block_size, head_dim]``.  A group with a window gives pages
back as soon as the window has passed them; all pages and the state slot go back when the
request ends.  Appending is all-or-nothing across groups and requests.

Host bookkeeping is separate from the device pools, so it runs (and is tested) without a GPU.
AxiomOperator/rllm: crates/rllm-kv/src/lib.rs:76-133 (SeqKv: block table, append -> slots,
all-or-nothing), crates/rllm-model/src/lib.rs:100-103,135-138 (one cache layout per group).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..parts.base import PagedKVNeed, StateNeed
from .allocator import BlockAllocator, OutOfPages, SlotAllocator


@dataclass
class PagedKVView:
    """What an attention-like mixer gets for one run entry in one step."""
    k: torch.Tensor              # [pages, kv_heads, block_size, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor    # int32 [requests in step, width]
    slots: torch.Tensor          # int32 [tokens in step]: page * block_size + offset of each new token
    block_size: int
    write: bool = True
    group: int = 0


@dataclass
class StateView:
    """What a mixer with fixed-size state gets: its plane of the state array and, per request of
    the step, the slot that holds the request's state."""
    state: torch.Tensor          # [max_requests, *shape]
    slots: torch.Tensor          # int32 [requests in step]
    write: bool = True


@dataclass
class _Request:
    length: int = 0
    tables: list = field(default_factory=list)     # per paged group: page id or None per logical block
    state_slot: Optional[int] = None


class PagedGroup:
    def __init__(self, need: PagedKVNeed, entries: list, n_blocks: int, block_size: int):
        self.need, self.entries, self.block_size, self.n_blocks = need, entries, block_size, n_blocks
        self.allocator = BlockAllocator(n_blocks)
        self.pool = None                               # device tensor, see CacheManager.allocate_device

    def first_needed_block(self, length: int) -> int:
        """Logical index of the first block that tokens at positions >= length can still read."""
        if self.need.window <= 0:
            return 0
        return max(0, length + 1 - self.need.window) // RELEASE_ALIGN * RELEASE_ALIGN // self.block_size


# Pages of a windowed group are given back in runs of this many keys: the attention kernels round
# the start of a window down to their key tile (at most 128 keys) and load whole tiles, so a page
# goes to another request only when no tile that is still read touches it.
RELEASE_ALIGN = 128


class RequestTooLong(ValueError):
    """A request would hold more tokens than the model's positions reach; nothing was taken."""

    def __init__(self, length, limit):
        self.length, self.limit = length, limit
        super().__init__(f"a request would hold {length} tokens, more than the {limit} positions the model "
                         f"has (max_position_embeddings)")


class StateGroup:
    def __init__(self, need: StateNeed, entries: list, max_requests: int):
        self.need, self.entries = need, entries
        self.state = None                              # [entry, max_requests, *shape]


class CacheManager:
    """`needs[i]` is the need of run entry i (PagedKVNeed, StateNeed or None); `cache_of[i]` names
    the earlier entry whose cache entry i reads instead of owning one (None: its own)."""

    def __init__(self, needs: Sequence, cache_of: Sequence, block_size: int, max_tokens: int,
                 max_requests: int, max_step_tokens: Optional[int] = None):
        """max_step_tokens: the most tokens of one request that a step brings, if the caller keeps to
        one (a scheduler's portion size).  A group whose layers read a window of keys only then gets a
        smaller pool: a request never holds more of its pages than the window, a step's tokens and the
        alignment of the release take (see RELEASE_ALIGN).  None: every group has pages for max_tokens."""
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.block_size = block_size
        self.max_requests = max_requests
        self.n_blocks = -(-max_tokens // block_size)
        self.paged: list[PagedGroup] = []
        self.stateful: list[StateGroup] = []
        self.entry_place: list = []                   # per run entry: ('kv', group, plane) | ('state', g, plane) | None
        for i, need in enumerate(needs):
            owner = cache_of[i]
            if owner is not None:
                if not 0 <= owner < i or cache_of[owner] is not None:
                    raise ValueError(f"run entry {i}: cache_of must name an earlier entry that owns a cache")
                if needs[owner] != need:
                    raise ValueError(f"run entry {i} reads the cache of entry {owner} but needs {need}, "
                                     f"not {needs[owner]}")
                self.entry_place.append(self.entry_place[owner])
                continue
            if need is None:
                self.entry_place.append(None)
            elif isinstance(need, PagedKVNeed):
                g = next((j for j, grp in enumerate(self.paged) if grp.need == need), None)
                if g is None:
                    self.paged.append(PagedGroup(need, [], self._group_blocks(need, max_step_tokens), block_size))
                    g = len(self.paged) - 1
                self.paged[g].entries.append(i)
                self.entry_place.append(("kv", g, len(self.paged[g].entries) - 1))
            elif isinstance(need, StateNeed):
                g = next((j for j, grp in enumerate(self.stateful) if grp.need == need), None)
                if g is None:
                    self.stateful.append(StateGroup(need, [], max_requests))
                    g = len(self.stateful) - 1
                self.stateful[g].entries.append(i)
                self.entry_place.append(("state", g, len(self.stateful[g].entries) - 1))
            else:
                raise TypeError(f"run entry {i}: unknown cache need {need!r}")
        self.cache_of = list(cache_of)
        self.slots = SlotAllocator(max_requests)
        self.requests: dict = {}
        self.max_length = 0          # most tokens a request may hold (0: no limit); see set_max_length

    def _group_blocks(self, need: PagedKVNeed, max_step_tokens) -> int:
        if need.window <= 0 or max_step_tokens is None:
            return self.n_blocks
        per_request = -(-(need.window + int(max_step_tokens) + RELEASE_ALIGN) // self.block_size) + 1
        return min(self.n_blocks, self.max_requests * per_request)

    def set_max_length(self, n: int) -> None:
        """Appends that would take a request beyond `n` tokens raise RequestTooLong (0: no limit)."""
        self.max_length = int(n)

    # ------------------------------------------------------------------ device side
    def allocate_device(self, device, dtype) -> None:
        for grp in self.paged:
            n = grp.need
            grp.pool = torch.zeros((len(grp.entries), 2, grp.n_blocks, n.num_kv_heads, self.block_size,
                                    n.head_dim), dtype=dtype, device=device)
        for grp in self.stateful:
            # one slot more than requests: the last one belongs to nobody; the padding rows of a step
            # that is replayed from a CUDA graph read and write it
            grp.state = torch.zeros((len(grp.entries), self.max_requests + 1, *grp.need.shape),
                                    dtype=grp.need.dtype, device=device)

    def device_bytes(self) -> int:
        total = 0
        for grp in self.paged:
            if grp.pool is not None:
                total += grp.pool.numel() * grp.pool.element_size()
        for grp in self.stateful:
            if grp.state is not None:
                total += grp.state.numel() * grp.state.element_size()
        return total

    def bytes_per_token(self, element_size: int) -> int:
        return sum(2 * len(g.entries) * g.need.num_kv_heads * g.need.head_dim * element_size
                   for g in self.paged)

    # ------------------------------------------------------------------ requests
    def has(self, rid) -> bool:
        return rid in self.requests

    def length(self, rid) -> int:
        return self.requests[rid].length

    def add_request(self, rid) -> None:
        """Registers a request and takes its state slot (zeroing the state if there is any)."""
        if rid in self.requests:
            raise ValueError(f"request {rid!r} is already live")
        slot = self.slots.take()
        self.requests[rid] = _Request(0, [[] for _ in self.paged], slot)
        for grp in self.stateful:
            if grp.state is not None:
                grp.state[:, slot].zero_()

    def free(self, rid) -> None:
        """Gives back every page and the state slot of a request."""
        req = self.requests.pop(rid)
        for grp, table in zip(self.paged, req.tables):
            for b in table:
                if b is not None:
                    grp.allocator.release(b)
        self.slots.give_back(req.state_slot)

    def pages_needed(self, rid, n_new: int) -> list:
        """New pages per paged group for `n_new` more tokens of request `rid` (0 tokens for an
        unknown request means a fresh one)."""
        req = self.requests.get(rid)
        length = req.length if req else 0
        out = []
        for gi, grp in enumerate(self.paged):
            have = len(req.tables[gi]) if req else 0
            out.append(max(0, -(-(length + n_new) // self.block_size) - have))
        return out

    def can_append(self, items: Sequence) -> bool:
        """`items`: (rid, n_new) pairs, each request at most once."""
        if self.max_length > 0 and any((self.requests[rid].length if rid in self.requests else 0) + n_new
                                       > self.max_length for rid, n_new in items):
            return False
        need = [0] * len(self.paged)
        new_requests = 0
        for rid, n_new in items:
            if rid not in self.requests:
                new_requests += 1
            for gi, p in enumerate(self.pages_needed(rid, n_new)):
                need[gi] += p
        if new_requests > self.slots.n_free:
            return False
        return all(n <= grp.allocator.n_free for n, grp in zip(need, self.paged))

    def check_append(self, items: Sequence) -> None:
        """Raises OutOfPages (or RequestTooLong) if `items` cannot all be appended; takes nothing."""
        if self.max_length > 0:
            for rid, n_new in items:
                length = (self.requests[rid].length if rid in self.requests else 0) + n_new
                if length > self.max_length:
                    raise RequestTooLong(length, self.max_length)
        need = [0] * len(self.paged)
        new_requests = sum(1 for rid, _ in items if rid not in self.requests)
        for rid, n_new in items:
            for gi, p in enumerate(self.pages_needed(rid, n_new)):
                need[gi] += p
        if new_requests > self.slots.n_free:
            raise OutOfPages(new_requests, self.slots.n_free, "state slots")
        for n, grp in zip(need, self.paged):
            if n > grp.allocator.n_free:
                raise OutOfPages(n, grp.allocator.n_free)

    def append(self, rid, n_new: int) -> list:
        """Grows request `rid` by `n_new` tokens.  Returns, per paged group, the slot
        (page * block_size + offset) of each new token.  All-or-nothing."""
        if n_new <= 0:
            raise ValueError("append needs at least one token")
        self.check_append([(rid, n_new)])
        if rid not in self.requests:
            self.add_request(rid)
        req = self.requests[rid]
        bs = self.block_size
        out = []
        for gi, grp in enumerate(self.paged):
            table = req.tables[gi]
            table.extend(grp.allocator.alloc(self.pages_needed(rid, n_new)[gi]))
            out.append([table[p // bs] * bs + p % bs for p in range(req.length, req.length + n_new)])
        req.length += n_new
        return out

    def release_passed(self, rid) -> int:
        """Gives back the pages of windowed groups that no later token of `rid` can read.
        Returns the number of pages released."""
        req = self.requests[rid]
        released = 0
        for gi, grp in enumerate(self.paged):
            first = grp.first_needed_block(req.length)
            table = req.tables[gi]
            for b in range(min(first, len(table))):
                if table[b] is not None:
                    grp.allocator.release(table[b])
                    table[b] = None
                    released += 1
        return released

    def truncate(self, rid, length: int) -> None:
        """Drops the tokens after `length`, releasing whole trailing pages.  Only for groups
        without a window (a windowed group may already have dropped earlier pages)."""
        req = self.requests[rid]
        if length > req.length:
            raise ValueError("truncate cannot grow a request")
        keep = -(-length // self.block_size)
        for gi, grp in enumerate(self.paged):
            table = req.tables[gi]
            while len(table) > keep:
                b = table.pop()
                if b is not None:
                    grp.allocator.release(b)
        req.length = length

    def block_table(self, rid, group: int) -> list:
        """Page per logical block; pages already given back read as 0.  No kernel dereferences
        them: pages are released in runs of RELEASE_ALIGN keys, the largest key tile, so every
        tile that still holds a key inside the window lies wholly in pages the request holds."""
        return [0 if b is None else b for b in self.requests[rid].tables[group]]

    def state_slot(self, rid) -> int:
        return self.requests[rid].state_slot

    def n_free_pages(self, group: int = 0) -> int:
        return self.paged[group].allocator.n_free if self.paged else 0

    # ------------------------------------------------------------------ invariants (tests)
    def check_invariants(self) -> None:
        """No page lost, held twice, or both free and held."""
        for gi, grp in enumerate(self.paged):
            held = []
            for req in self.requests.values():
                held += [b for b in req.tables[gi] if b is not None]
            if len(held) != len(set(held)):
                raise AssertionError(f"group {gi}: a page is held twice")
            free = grp.allocator._free
            if len(free) != len(set(free)):
                raise AssertionError(f"group {gi}: a page is in the free list twice")
            if set(free) & set(held):
                raise AssertionError(f"group {gi}: a page is both free and held")
            if len(free) + len(held) != grp.allocator.n_blocks:
                raise AssertionError(f"group {gi}: {grp.allocator.n_blocks - len(free) - len(held)} pages lost")
        slots = [r.state_slot for r in self.requests.values()]
        if len(slots) != len(set(slots)):
            raise AssertionError("a state slot is held twice")
        if len(slots) + self.slots.n_free != self.max_requests:
            raise AssertionError("a state slot is lost")
