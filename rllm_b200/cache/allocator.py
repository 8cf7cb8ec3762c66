"""Page and slot allocators (host side, no device work).

`BlockAllocator` hands out fixed-size pages from a free list, lowest ids first, all or none,
with reference counts; giving back a page that is not held is an error, never a silent
double free.  AxiomOperator/rllm: crates/rllm-kv/src/lib.rs:17-74 (free list built reversed
and popped from the back, `alloc_n` all-or-none, `share` / `release`).
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """Not enough free pages (or slots); nothing was taken."""

    def __init__(self, need, free, what="pages"):
        self.need, self.free, self.what = need, free, what
        super().__init__(f"out of {what}: need {need}, {free} free")


class BlockAllocator:
    def __init__(self, n_blocks: int):
        if n_blocks < 0:
            raise ValueError("n_blocks must be >= 0")
        self.n_blocks = n_blocks
        self._free = list(range(n_blocks - 1, -1, -1))      # pop() yields the lowest id
        self._ref = [0] * n_blocks

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> list:
        """Takes `n` pages or raises OutOfPages without taking any."""
        if n > len(self._free):
            raise OutOfPages(n, len(self._free))
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self._ref[b] = 1
        return out

    def share(self, block: int) -> None:
        if self._ref[block] <= 0:
            raise ValueError(f"page {block} is not held and cannot be shared")
        self._ref[block] += 1

    def release(self, block: int) -> None:
        if not 0 <= block < self.n_blocks or self._ref[block] <= 0:
            raise ValueError(f"page {block} is not held (freed twice?)")
        self._ref[block] -= 1
        if self._ref[block] == 0:
            self._free.append(block)

    def refcount(self, block: int) -> int:
        return self._ref[block]

    def held(self) -> list:
        return [b for b, r in enumerate(self._ref) if r > 0]


class SlotAllocator:
    """Slots for fixed-size per-request state: one per live request."""

    def __init__(self, n_slots: int):
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._held = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages(1, 0, "state slots")
        s = self._free.pop()
        self._held.add(s)
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._held:
            raise ValueError(f"state slot {slot} is not held (freed twice?)")
        self._held.remove(slot)
        self._free.append(slot)
