"""The cache manager and step builder of the C++ host runtime (``csrc/host_runtime.cpp``) behind
the interface of :class:`~rllm_b200.cache.manager.CacheManager`.

The grouping of run entries (which entries share a page pool, which read another entry's cache)
is decided once in Python, exactly as in ``CacheManager``; everything that happens per step --
page accounting, block tables, slots, window release, and the flattening of a step's items into
the int32 arrays the kernels read -- runs in C++ and writes into the engine's pinned staging
buffer.  Request ids of any hashable type are mapped to 64-bit handles here.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_int32, c_int64, c_void_p
from typing import Sequence

import numpy as np
import torch

from ..csrc import build
from .allocator import OutOfPages
from .manager import CacheManager, RequestTooLong

OK, ERR_OUT_OF_PAGES, ERR_OUT_OF_SLOTS, ERR_UNKNOWN_REQUEST, ERR_BAD_ARG, ERR_DOUBLE_FREE, ERR_INVARIANT, \
    ERR_LIVE_TWICE, ERR_BUFFER, ERR_TOO_LONG = range(10)

_lib = None


def host_lib():
    global _lib
    if _lib is None:
        lib = build.load("host")
        lib.rllm_cache_create.restype = c_void_p
        lib.rllm_cache_create.argtypes = [c_int, POINTER(c_int), c_int, c_int, c_int, POINTER(c_int)]
        lib.rllm_cache_destroy.argtypes = [c_void_p]
        for name in ("has", "length", "state_slot"):
            getattr(lib, f"rllm_cache_{name}").argtypes = [c_void_p, c_int64]
        lib.rllm_cache_n_requests.argtypes = [c_void_p]
        lib.rllm_cache_set_max_length.argtypes = [c_void_p, c_int]
        lib.rllm_cache_n_free_pages.argtypes = [c_void_p, c_int]
        lib.rllm_cache_n_free_slots.argtypes = [c_void_p]
        lib.rllm_cache_pages_needed.argtypes = [c_void_p, c_int64, c_int, POINTER(c_int)]
        lib.rllm_cache_check_append.argtypes = [c_void_p, c_int, POINTER(c_int64), POINTER(c_int)]
        lib.rllm_cache_last_refusal.argtypes = [c_void_p, POINTER(c_int), POINTER(c_int)]
        lib.rllm_cache_add_request.argtypes = [c_void_p, c_int64]
        lib.rllm_cache_append.argtypes = [c_void_p, c_int64, c_int, POINTER(c_int), POINTER(c_int)]
        lib.rllm_cache_release_passed.argtypes = [c_void_p, c_int64, POINTER(c_int)]
        lib.rllm_cache_free.argtypes = [c_void_p, c_int64]
        lib.rllm_cache_truncate.argtypes = [c_void_p, c_int64, c_int]
        lib.rllm_cache_check_invariants.argtypes = [c_void_p]
        lib.rllm_cache_block_table.argtypes = [c_void_p, c_int64, c_int, POINTER(c_int), c_int, c_int]
        lib.rllm_step_build.argtypes = [c_void_p, c_int, POINTER(c_int64), POINTER(c_int), POINTER(c_int),
                                        POINTER(c_int), POINTER(c_int), c_int, c_int, c_int, c_int, c_void_p, c_int,
                                        POINTER(c_int), POINTER(c_int), POINTER(c_int)]
        _lib = lib
    return _lib


def _ip(a: np.ndarray):
    return a.ctypes.data_as(POINTER(c_int))


class _Slots:
    def __init__(self, owner):
        self._o = owner

    @property
    def n_free(self) -> int:
        return host_lib().rllm_cache_n_free_slots(self._o._h)


class NativeCacheManager(CacheManager):
    """Same construction and interface as CacheManager; the bookkeeping lives in C++."""

    def __init__(self, needs: Sequence, cache_of: Sequence, block_size: int, max_tokens: int, max_requests: int,
                 max_step_tokens=None):
        super().__init__(needs, cache_of, block_size, max_tokens, max_requests, max_step_tokens)    # groups, entry_place
        lib = host_lib()
        windows = (c_int * max(1, len(self.paged)))(*[g.need.window for g in self.paged])
        group_blocks = (c_int * max(1, len(self.paged)))(*[g.n_blocks for g in self.paged])
        self._h = c_void_p(lib.rllm_cache_create(len(self.paged), windows, block_size, self.n_blocks, max_requests,
                                                 group_blocks))
        if not self._h:
            raise ValueError("cache manager: bad sizes")
        self._ids: dict = {}
        self._next = 1
        self.slots = _Slots(self)
        self.requests = self._ids            # truthiness and membership as in the Python manager

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                host_lib().rllm_cache_destroy(self._h)
                self._h = None
        except Exception:
            pass

    # ---- ids
    def _id(self, rid, create=False) -> int:
        h = self._ids.get(rid)
        if h is None:
            if not create:
                return 0
            h = self._ids[rid] = self._next
            self._next += 1
        return h

    def _raise(self, code: int, what: str):
        if code in (ERR_OUT_OF_PAGES, ERR_OUT_OF_SLOTS):
            need, free = c_int(), c_int()
            host_lib().rllm_cache_last_refusal(self._h, need, free)
            raise OutOfPages(need.value, free.value, "pages" if code == ERR_OUT_OF_PAGES else "state slots")
        if code == ERR_TOO_LONG:
            need, limit = c_int(), c_int()
            host_lib().rllm_cache_last_refusal(self._h, need, limit)
            raise RequestTooLong(need.value, limit.value)
        if code == ERR_UNKNOWN_REQUEST:
            raise KeyError(what)
        if code == ERR_DOUBLE_FREE:
            raise ValueError(f"{what}: a page is not held (freed twice?)")
        if code == ERR_LIVE_TWICE:
            raise ValueError(f"{what}: request is already live")
        if code == ERR_INVARIANT:
            raise AssertionError(f"{what}: cache invariants violated")
        raise ValueError(f"{what}: bad argument")

    # ---- interface of CacheManager
    def set_max_length(self, n: int) -> None:
        self.max_length = int(n)
        host_lib().rllm_cache_set_max_length(self._h, int(n))

    def has(self, rid) -> bool:
        return rid in self._ids

    def length(self, rid) -> int:
        n = host_lib().rllm_cache_length(self._h, self._ids[rid])
        if n < 0:
            raise KeyError(rid)
        return n

    def add_request(self, rid) -> None:
        if rid in self._ids:
            raise ValueError(f"request {rid!r} is already live")
        st = host_lib().rllm_cache_add_request(self._h, self._id(rid, create=True))
        if st:
            del self._ids[rid]
            self._raise(st, f"add_request({rid!r})")
        self._zero_state(rid)

    def _zero_state(self, rid) -> None:
        slot = self.state_slot(rid)
        for grp in self.stateful:
            if grp.state is not None:
                grp.state[:, slot].zero_()

    def free(self, rid) -> None:
        h = self._ids.pop(rid)               # KeyError for an unknown request, as the Python manager
        st = host_lib().rllm_cache_free(self._h, h)
        if st:
            self._raise(st, f"free({rid!r})")

    def pages_needed(self, rid, n_new: int) -> list:
        out = (c_int * max(1, len(self.paged)))()
        host_lib().rllm_cache_pages_needed(self._h, self._ids.get(rid, 0), n_new, out)
        return list(out)[:len(self.paged)]

    def _check(self, items):
        n = len(items)
        rids = np.fromiter((self._ids.get(r, -(i + 1)) for i, (r, _) in enumerate(items)), np.int64, n)
        cnt = np.fromiter((k for _, k in items), np.int32, n)
        return host_lib().rllm_cache_check_append(self._h, n, rids.ctypes.data_as(POINTER(c_int64)), _ip(cnt))

    def can_append(self, items: Sequence) -> bool:
        return self._check(list(items)) == OK

    def check_append(self, items: Sequence) -> None:
        st = self._check(list(items))
        if st:
            self._raise(st, "append")

    def append(self, rid, n_new: int) -> list:
        if n_new <= 0:
            raise ValueError("append needs at least one token")
        known = rid in self._ids
        G = len(self.paged)
        slots = np.empty(max(1, G * n_new), np.int32)
        is_new = c_int()
        st = host_lib().rllm_cache_append(self._h, self._id(rid, create=True), n_new, _ip(slots), is_new)
        if st:
            if not known:
                del self._ids[rid]
            self._raise(st, f"append({rid!r})")
        if is_new.value:
            self._zero_state(rid)
        return [slots[g * n_new:(g + 1) * n_new].tolist() for g in range(G)]

    def release_passed(self, rid) -> int:
        out = c_int()
        st = host_lib().rllm_cache_release_passed(self._h, self._ids[rid], out)
        if st:
            self._raise(st, f"release_passed({rid!r})")
        return out.value

    def truncate(self, rid, length: int) -> None:
        st = host_lib().rllm_cache_truncate(self._h, self._ids[rid], length)
        if st:
            self._raise(st, f"truncate({rid!r})")

    def block_table(self, rid, group: int, raw: bool = False) -> list:
        cap = self.n_blocks + 1
        buf = (c_int * cap)()
        n = host_lib().rllm_cache_block_table(self._h, self._ids[rid], group, buf, cap, 1 if raw else 0)
        if n < 0:
            raise KeyError(rid)
        out = list(buf)[:n]
        return [None if b < 0 else b for b in out] if raw else out

    def state_slot(self, rid) -> int:
        return host_lib().rllm_cache_state_slot(self._h, self._ids[rid])

    def n_free_pages(self, group: int = 0) -> int:
        return host_lib().rllm_cache_n_free_pages(self._h, group) if self.paged else 0

    def check_invariants(self) -> None:
        st = host_lib().rllm_cache_check_invariants(self._h)
        if st:
            raise AssertionError("cache invariants violated: a page or slot is lost, held twice or both free and held")
        if host_lib().rllm_cache_n_requests(self._h) != len(self._ids):
            raise AssertionError("request handles out of step with the native cache")

    # ---- the step builder
    def build_step(self, items, vocab: int, out: torch.Tensor, pad_requests: int = 0, pad_width: int = 0,
                   pad_quantum: int = 0):
        """Appends the items and writes the step's arrays into the pinned int32 tensor `out`.
        Returns (offsets, meta = (n, R, m, width, total, longest), new_request_flags) or raises;
        returns (None, meta, None) when `out` is too small (nothing appended; meta's total tells the
        size needed).  pad_quantum: block tables as wide as the longest request rounded up to that
        many tokens (the padded shape of a captured decode step)."""
        n_items = len(items)
        ids = self._ids
        created = []
        rids = np.empty(n_items, np.int64)
        for i, it in enumerate(items):
            h = ids.get(it.request_id)
            if h is None:
                created.append(it.request_id)
                h = self._id(it.request_id, create=True)
            rids[i] = h
        try:
            if all(len(it.tokens) == 1 for it in items):          # decode steps: no per-item arrays
                n_tok = np.ones(n_items, np.int32)
                toks = np.fromiter((it.tokens[0] for it in items), np.int64, n_items)
            else:
                n_tok = np.fromiter((len(it.tokens) for it in items), np.int32, n_items)
                toks = np.concatenate([np.asarray(it.tokens, np.int64) for it in items]) if n_items else np.empty(0, np.int64)
            if toks.size and (toks.min() < 0 or toks.max() >= vocab):
                raise ValueError
            toks = toks.astype(np.int32)
            n_want = np.fromiter((len(it.want) for it in items), np.int32, n_items)
            want = np.fromiter((w for it in items for w in it.want), np.int32, int(n_want.sum()))
        except (ValueError, TypeError):
            for r in created:
                del self._ids[r]
            raise ValueError("bad token ids or wanted places")
        G = len(self.paged)
        offsets = (c_int * (7 + 2 * G))()
        meta = (c_int * 6)()
        flags = (c_int * max(1, n_items))()
        st = host_lib().rllm_step_build(self._h, n_items, rids.ctypes.data_as(POINTER(c_int64)), _ip(n_tok), _ip(toks),
                                        _ip(n_want), _ip(want), vocab, pad_requests, pad_width, pad_quantum,
                                        c_void_p(out.data_ptr()), out.numel(), offsets, meta, flags)
        if st:
            for r in created:
                del self._ids[r]
            if st == ERR_BUFFER:
                return None, tuple(meta), None
            self._raise(st, "step")
        if self.stateful:
            for i, it in enumerate(items):
                if flags[i]:
                    self._zero_state(it.request_id)
        return list(offsets), tuple(meta), list(flags)[:n_items]
