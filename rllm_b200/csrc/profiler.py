"""Per-launcher device timing behind an environment switch.

With ``RLLM_B200_PROFILE=1`` every call of an extern "C" launcher (`rllm_skinny_gemm`,
`rllm_paged_flash_attention`, ...) is bracketed by a pair of CUDA events on the launching stream.
The pairs are resolved in batches (never a synchronize per launch), summed per launcher, and a
table -- calls, total and mean device time, share, and the span from the first launch to the last
-- is printed to standard error when the process ends or when :func:`report` is called.  The
engine does not capture CUDA graphs while the switch is on (events cannot be recorded into a
capture), so the numbers are those of eager launches: read shares, not the step time.

The reference has the same switch: an event pair around every launch, resolved in batches, totals
and the first-to-last span printed when the backend is dropped, graphs off meanwhile
(crates/rllm-cuda/src/backend.rs:275-285, 630-674, 1252-1269).
"""
from __future__ import annotations

import atexit
import os
import sys
from collections import defaultdict

import torch

_RESOLVE_EVERY = 2048            # pending pairs before a batch is resolved (one synchronize per batch)


def enabled() -> bool:
    return os.environ.get("RLLM_B200_PROFILE", "0") not in ("", "0")


class Profile:
    def __init__(self):
        self.total_ms = defaultdict(float)
        self.calls = defaultdict(int)
        self.pending: list = []
        self.first = None
        self.last = None

    def timed(self, name, fn):
        def call(*args):
            start = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            start.record()
            status = fn(*args)
            end.record()
            if self.first is None:
                self.first = start
            self.last = end
            self.pending.append((name, start, end))
            if len(self.pending) >= _RESOLVE_EVERY:
                self.resolve()
            return status
        return call

    def resolve(self) -> None:
        if not self.pending:
            return
        self.pending[-1][2].synchronize()
        for name, start, end in self.pending:
            self.total_ms[name] += start.elapsed_time(end)
            self.calls[name] += 1
        self.pending.clear()

    def rows(self) -> list:
        """[(launcher, calls, total ms, mean us, share)] by falling total."""
        self.resolve()
        whole = sum(self.total_ms.values()) or 1.0
        return [(n, self.calls[n], t, 1e3 * t / self.calls[n], t / whole)
                for n, t in sorted(self.total_ms.items(), key=lambda kv: -kv[1])]

    def span_ms(self) -> float:
        if self.first is None:
            return 0.0
        self.last.synchronize()
        return self.first.elapsed_time(self.last)

    def report(self, file=None) -> None:
        file = file or sys.stderr
        rows = self.rows()
        if not rows:
            return
        print("[rllm_b200 profile] launcher                          calls   total ms   mean us   share", file=file)
        for name, calls, total, mean, share in rows:
            print(f"[rllm_b200 profile] {name:<32} {calls:>7} {total:>10.3f} {mean:>9.2f} {100 * share:>6.1f}%",
                  file=file)
        busy = sum(r[2] for r in rows)
        print(f"[rllm_b200 profile] kernels {busy:.3f} ms inside a span of {self.span_ms():.3f} ms "
              "(eager launches, graphs off)", file=file)

    def reset(self) -> None:
        self.resolve()
        self.total_ms.clear()
        self.calls.clear()
        self.first = self.last = None


_profile = None


def profile() -> Profile:
    global _profile
    if _profile is None:
        _profile = Profile()
        atexit.register(_at_exit)
    return _profile


def _at_exit() -> None:
    try:
        _profile.report()
    except Exception:                 # the CUDA context may be gone already
        pass


def report(file=None) -> None:
    if _profile is not None:
        _profile.report(file)


class TimedLibrary:
    """A loaded library whose launchers (functions that return a launch status) are timed."""

    # entry points that launch nothing
    UNTIMED = ("rllm_paged_flash_decode_static_error",)

    def __init__(self, lib):
        self._lib = lib
        self._cache: dict = {}

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not name.startswith("rllm_") or name in self.UNTIMED:
            return fn
        wrapped = self._cache.get(name)
        if wrapped is None:
            wrapped = self._cache[name] = profile().timed(name, fn)
        return wrapped
