"""Python wrappers over the extern "C" kernel launchers.

Every wrapper takes CUDA torch tensors, checks what the kernel assumes (device,
dtype, contiguity, sizes) and launches on the current torch stream.  There is no
CPU or library fallback: a tensor that is not on a CUDA device, or a library that
cannot be built and loaded, raises.
"""
from __future__ import annotations

import ctypes
import os
import struct
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build, profiler

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {t.dtype}; kernels take float32 and bfloat16") from None


def _ptr(t):
    if t is None:
        return c_void_p(0)
    if _trace is not None:
        _trace.keep.append(t)                 # a traced launch names this memory: it stays alive with the trace
    return c_void_p(t.data_ptr())


# ------------------------------------------------------------------ trace and replay of launches
# A step that is not replayed from a CUDA graph launches its kernels from Python, and most of what a
# launch costs the host is the wrapper around it: checks, dispatch rules, argument conversion (7 to
# 13 us against 3.5 us for the call itself).  The layers of a model are alike: what one layer launches,
# the next launches too, with its own weights and cache planes in place of the first one's.  So the
# launches of one layer are recorded (`tracing`) and replayed for the layers of the same build
# (`Trace.replay`): the recorded calls again, argument for argument, with the pointers that belong to
# the layer swapped.  Whatever a wrapper decides from shapes and types it has decided once.
_trace = None


class Trace:
    """The launches recorded between `tracing()` and its end: (launcher, arguments) in order.
    `freeze(addresses)` names the addresses that belong to the layer, in the order in which
    `replay(addresses of another layer)` gives theirs; the calls then live in the C++ host runtime
    (host_runtime.cpp, rllm_trace_replay), which makes them again through the launchers'
    packed-argument forms, one call from Python for the whole layer."""

    def __init__(self):
        self.calls: list = []             # [library, launcher name, [ctypes arguments]]
        self.keep: list = []              # tensors (and ctypes objects) whose memory the arguments name
        self.own_launches = 0
        self._native = None
        self._n_roles = 0

    @staticmethod
    def _word(a) -> int:
        if isinstance(a, c_void_p):
            return a.value or 0
        if isinstance(a, c_float):
            return struct.unpack("<I", struct.pack("<f", a.value))[0]
        if isinstance(a, (c_int, c_longlong)):
            return a.value & 0xFFFFFFFFFFFFFFFF
        if isinstance(a, int):
            return a & 0xFFFFFFFFFFFFFFFF
        return ctypes.cast(a, c_void_p).value or 0          # byref(...) of an out parameter, a ctypes pointer

    def freeze(self, addresses) -> None:
        role_of = {}
        for i, addr in enumerate(addresses):
            role_of.setdefault(addr, i)
        self._n_roles = len(addresses)
        fns, n_args, words, swap_at, swap_role = [], [], [], [], []
        for lib, name, args in self.calls:
            fn = getattr(lib, name + "_packed")
            fns.append(ctypes.cast(fn, c_void_p).value)
            n_args.append(len(args))
            for a in args:
                if isinstance(a, c_void_p) and a.value in role_of:
                    swap_at.append(len(words))
                    swap_role.append(role_of[a.value])
                words.append(self._word(a))
        self.keep.append([a for _, _, args in self.calls for a in args])     # out parameters stay alive
        host = build.load("host")
        host.rllm_trace_create.restype = c_void_p
        host.rllm_trace_create.argtypes = [c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int),
                                           ctypes.POINTER(ctypes.c_ulonglong), c_int, ctypes.POINTER(c_int),
                                           ctypes.POINTER(c_int)]
        host.rllm_trace_replay.argtypes = [c_void_p, ctypes.POINTER(ctypes.c_ulonglong), c_int, ctypes.POINTER(c_int)]
        host.rllm_trace_destroy.argtypes = [c_void_p]
        n = len(fns)
        self._host = host
        self._native = host.rllm_trace_create(
            n, (c_void_p * max(n, 1))(*fns), (c_int * max(n, 1))(*n_args),
            (ctypes.c_ulonglong * max(len(words), 1))(*words), len(swap_at),
            (c_int * max(len(swap_at), 1))(*swap_at), (c_int * max(len(swap_role), 1))(*swap_role))
        if not self._native:
            raise KernelError("the host runtime refused a trace of launches")

    def replay(self, addresses) -> None:
        """Launches the recorded calls again with `addresses` (same order as at `freeze`) in place."""
        if len(addresses) != self._n_roles:
            raise KernelError("replay: other addresses than the trace was frozen with")
        failed = c_int(-1)
        status = self._host.rllm_trace_replay(self._native, (ctypes.c_ulonglong * max(self._n_roles, 1))(*addresses),
                                              self._n_roles, ctypes.byref(failed))
        if status:
            name = self.calls[failed.value][1] if 0 <= failed.value < len(self.calls) else "?"
            raise KernelError(f"replayed launch {name}: status {status}")
        add_launches(self.own_launches)

    def __del__(self):
        try:
            if self._native:
                self._host.rllm_trace_destroy(self._native)
                self._native = None
        except Exception:
            pass


class _RecordingLibrary:
    def __init__(self, lib, trace):
        self._lib, self._trace = lib, trace

    def __getattr__(self, name):
        lib, trace = self._lib, self._trace
        fn = getattr(lib, name)

        def call(*args):
            trace.calls.append((lib, name, list(args)))
            return fn(*args)
        return call


class tracing:
    """``with ops.tracing() as trace:`` every launch inside is recorded into `trace` (and made)."""

    def __enter__(self):
        global _trace
        if _trace is not None:
            raise KernelError("a trace is being recorded already")
        _trace = Trace()
        self._before = _launches
        return _trace

    def __exit__(self, *exc):
        global _trace
        trace, _trace = _trace, None
        trace.own_launches = _launches - self._before


class untraced:
    """``with ops.untraced():`` launches inside are made but not recorded (what one pass does once for
    all its layers, like the table of rotary angles)."""

    def __enter__(self):
        global _trace
        self._saved, _trace = _trace, None

    def __exit__(self, *exc):
        global _trace
        _trace = self._saved


def can_trace() -> bool:
    """Launches can be recorded (not while every launch is timed with events)."""
    return not profiler.enabled()


_raw_stream = torch._C._cuda_getCurrentRawStream
_current_device = torch._C._cuda_getDevice


def _stream():
    """The current stream of the current device, as the launchers take it (the raw handle: building a
    torch.cuda.Stream object for every launch costs more than the launch)."""
    return c_void_p(_raw_stream(_current_device()))


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("rllm_b200 kernels run on a CUDA device only; got a tensor on "
                              f"{t.device}. There is no CPU path.")


def _need_contig(**ts):
    for name, t in ts.items():
        if t is not None and not t.is_contiguous():
            raise KernelError(f"{name} must be contiguous")


_launches = 0


def launch_count() -> int:
    """Number of this package's own kernels launched so far (library products not counted)."""
    return _launches


def add_launches(n: int) -> None:
    """Counts kernels that ran from a replayed CUDA graph."""
    global _launches
    _launches += n


def _check(status: int, what: str, own: bool = True):
    global _launches
    if status != 0:
        raise KernelError(f"{what}: CUDA error {status} (cudaError_t)")
    if own:
        _launches += 1


_timed: dict = {}


def _lib(name: str):
    """The loaded library `name`; with RLLM_B200_PROFILE=1 its launchers are timed with CUDA events."""
    lib = _timed.get(name)
    if lib is None:
        lib = build.load(name)
        if profiler.enabled():
            lib = profiler.TimedLibrary(lib)
        _timed[name] = lib
    if _trace is not None:
        return _RecordingLibrary(lib, _trace)
    return lib


def core():
    return _lib("core")


# ------------------------------------------------------------------ elementwise

def embed(table, tokens, out, err=None):
    """out[t,:] = table[tokens[t],:] as float32.  table [V,d] f32/bf16, tokens int32 [n], out f32 [n,d]."""
    _need_cuda(table, tokens, out)
    _need_contig(table=table, tokens=tokens, out=out)
    n, d = out.shape
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32 and table.shape[1] == d
    _check(core().rllm_embed(_ptr(table), _code(table), _ptr(tokens), _ptr(out), c_int(n), c_int(d),
                             c_int(table.shape[0]), _ptr(err), _stream()), "embed")
    return out


def add_rms_norm(x, delta, weight, out, eps, rows=None, write_x=True):
    """out[r] = rmsnorm(x[src] (+ delta[src])) * weight with src = rows[r] if rows is given else r.
    x is the float32 residual stream and receives the sum when write_x (and delta is given)."""
    _need_cuda(x, delta, weight, out, rows)
    _need_contig(x=x, delta=delta, weight=weight, out=out, rows=rows)
    d = x.shape[-1]
    n_rows = out.shape[0]
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == d
    assert out.shape[-1] == d
    if rows is None:
        assert x.shape[0] == n_rows
    else:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    if delta is not None:
        assert delta.shape == x.shape
    _check(core().rllm_add_rms_norm(_ptr(x), _ptr(delta), c_int(_code(delta) if delta is not None else F32),
                                    _ptr(rows), _ptr(weight), _ptr(out), c_int(_code(out)), c_int(n_rows),
                                    c_int(d), c_float(eps), c_int(1 if write_x else 0), _stream()),
           "add_rms_norm")
    return out


def add_inplace(x, delta):
    _need_cuda(x, delta)
    _need_contig(x=x, delta=delta)
    assert x.dtype == torch.float32 and x.shape == delta.shape
    _check(core().rllm_add_inplace(_ptr(x), _ptr(delta), c_int(_code(delta)), c_longlong(x.numel()),
                                   _stream()), "add_inplace")
    return x


def silu_mul(gate_up, out):
    """gate_up [n, 2F] (gate columns then up columns) -> out [n, F] = silu(gate) * up."""
    _need_cuda(gate_up, out)
    _need_contig(gate_up=gate_up, out=out)
    n, F = out.shape
    assert gate_up.shape == (n, 2 * F)
    _check(core().rllm_silu_mul(_ptr(gate_up), c_int(_code(gate_up)), _ptr(out), c_int(_code(out)),
                                c_int(n), c_int(F), _stream()), "silu_mul")
    return out


def rope_table(positions, inv_freq):
    """(cos, sin) of positions[t] * inv_freq[i] as float32 [n, head_dim/2, 2]: the rotation angles of a
    step's tokens, worked out once and read by every layer's qk_norm_rope_store."""
    _need_cuda(positions, inv_freq)
    n, half = positions.numel(), inv_freq.numel()
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
    out = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(core().rllm_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(out), c_int(n), c_int(half), _stream()),
           "rope_table")
    return out


def qk_norm_rope_store(qkv, q_norm_w, k_norm_w, inv_freq, positions, slots, q_out, k_cache, v_cache,
                       H, K, hd, block_size, eps, write_kv=True, cs_table=None):
    """Fused per-head q/k RMSNorm, rotary embedding and paged K/V write; see elementwise.cu.
    The rotation takes its angles from `cs_table` (rope_table: made once per step and shared by the
    layers); given `inv_freq` alone, the table is made here; neither: no rotation."""
    _need_cuda(qkv, q_norm_w, k_norm_w, inv_freq, positions, slots, q_out, k_cache, v_cache)
    _need_contig(qkv=qkv, q_out=q_out, k_cache=k_cache, v_cache=v_cache, positions=positions, slots=slots)
    n = qkv.shape[0]
    assert qkv.shape[1] == (H + 2 * K) * hd and q_out.shape == (n, H * hd)
    assert positions.dtype == torch.int32 and slots.dtype == torch.int32
    assert positions.numel() == n and slots.numel() == n
    if hd % 4 or hd > 256:
        raise KernelError(f"head size {hd} is not supported: the q/k norm + rotary kernel takes multiples of 4 up to 256")
    for w in (q_norm_w, k_norm_w):
        assert w is None or (w.dtype == torch.float32 and w.numel() == hd)
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == hd // 2)
    assert k_cache.dtype == q_out.dtype == v_cache.dtype
    if cs_table is None and inv_freq is not None:
        cs_table = rope_table(positions, inv_freq)
    assert cs_table is None or (cs_table.dtype == torch.float32 and cs_table.shape == (n, hd // 2, 2)
                                and cs_table.is_contiguous())
    _check(core().rllm_qk_norm_rope_store(
        _ptr(qkv), c_int(_code(qkv)), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cs_table), _ptr(positions),
        _ptr(slots), _ptr(q_out), c_int(_code(q_out)), _ptr(k_cache), _ptr(v_cache), c_int(_code(k_cache)),
        c_int(n), c_int(H), c_int(K), c_int(hd), c_int(block_size), c_float(eps),
        c_int(1 if write_kv else 0), c_longlong(k_cache.shape[0] * block_size), _ptr(error_word(qkv.device)),
        _stream()), "qk_norm_rope_store")
    return q_out


# ------------------------------------------------------------------ attention

def paged_attention_generic(q, k_cache, v_cache, out, positions, seq_ids, block_table, H, K, hd,
                            block_size, scale, window=0):
    """Plain paged causal attention; q/out [n, H*hd], caches [pages, K, block_size, hd]."""
    _need_cuda(q, k_cache, v_cache, out, positions, seq_ids, block_table)
    _need_contig(q=q, k_cache=k_cache, v_cache=v_cache, out=out, positions=positions, seq_ids=seq_ids)
    n = q.shape[0]
    assert q.shape == (n, H * hd) and out.shape == (n, H * hd)
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1
    assert positions.dtype == torch.int32 and seq_ids.dtype == torch.int32
    if hd > 512:
        raise KernelError(f"head size {hd} exceeds the attention kernel's limit of 512")
    if H % K:
        raise KernelError(f"{H} query heads are not a multiple of {K} key/value heads")
    _check(core().rllm_paged_attention_generic(
        _ptr(q), c_int(_code(q)), _ptr(k_cache), _ptr(v_cache), c_int(_code(k_cache)), _ptr(out),
        c_int(_code(out)), _ptr(positions), _ptr(seq_ids), _ptr(block_table), c_int(block_table.stride(0)),
        c_int(n), c_int(H), c_int(K), c_int(hd), c_int(block_size), c_float(scale), c_int(window),
        c_int(min(k_cache.shape[0], 0x7fffffff)), _ptr(error_word(q.device)), _stream()), "paged_attention_generic")
    return out


# ------------------------------------------------------------------ matrix products

def gemm_plain(a, w, out, accumulate=False):
    """out[m,n] (+)= a[m,k] . w[n,k]^T with float32 multiply-add on the CUDA cores."""
    _need_cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if accumulate and out.dtype != torch.float32:
        raise KernelError("accumulating product needs a float32 output")
    _check(core().rllm_gemm_plain(_ptr(a), c_int(_code(a)), _ptr(w), c_int(_code(w)), _ptr(out),
                                  c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
                                  c_int(w.stride(0)), c_int(out.stride(0)), c_int(1 if accumulate else 0),
                                  _stream()), "gemm_plain")
    return out


# ------------------------------------------------------------------ sampling

def logit_adjust(logits, index, delta):
    """logits.view(-1)[index[i]] += delta[i] in place (float32 logits, int64 index, float32 delta on
    the device; the positions must be distinct)."""
    _need_cuda(logits, index, delta)
    assert logits.dtype == torch.float32 and index.dtype == torch.int64 and delta.dtype == torch.float32
    assert index.numel() == delta.numel() and index.is_contiguous() and delta.is_contiguous()
    _check(core().rllm_logit_adjust(_ptr(logits), _ptr(index), _ptr(delta), c_int(index.numel()), _stream()),
           "logit_adjust")
    return logits


def sample_rows(logits, out_ids, temperature=None, top_k=None, top_p=None, seed=None, counter=None):
    """One token id per row of float32 logits [rows, vocab]; all parameter arrays are per row
    (float32, int32, float32, int64, int64) or None (greedy)."""
    _need_cuda(logits, out_ids, temperature, top_k, top_p, seed, counter)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert out_ids.dtype == torch.int32 and out_ids.numel() == rows
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32),
                  (seed, torch.int64), (counter, torch.int64)):
        assert t is None or (t.dtype == dt and t.numel() == rows and t.is_contiguous())
    if vocab >= 1 << 24:
        raise KernelError(f"vocabulary {vocab} exceeds the sampler's limit of 2^24 - 1")
    _check(core().rllm_sample_rows(_ptr(logits), c_longlong(logits.stride(0)), c_int(rows), c_int(vocab),
                                   _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seed), _ptr(counter),
                                   _ptr(out_ids), _stream()), "sample_rows")
    return out_ids


# ------------------------------------------------------------------ library product and dispatch

def gemm_lib(a, w, out, accumulate=False):
    """out[m,n] (+)= a[m,k] . w[n,k]^T through cuBLAS: bfloat16 operands, float32 accumulation."""
    _need_cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert w.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    st = _lib("blas").rllm_gemm_lib(_ptr(a), _ptr(w), _ptr(out), c_int(_code(out)), c_int(m), c_int(n),
                                          c_int(k), c_int(a.stride(0)), c_int(w.stride(0)),
                                          c_int(out.stride(0)), c_int(1 if accumulate else 0), _stream())
    if st >= 10000:
        raise KernelError(f"gemm_lib: cuBLAS status {st - 10000} for m={m} n={n} k={k}")
    _check(st, "gemm_lib", own=False)
    return out


EPI_STORE, EPI_ACCUM, EPI_SWIGLU = 0, 1, 2
SKINNY_MAX_ROWS = 64


def _skinny_ok(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] <= SKINNY_MAX_ROWS
            and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_gemm(a, w, out, epilogue=EPI_STORE, up_row_offset=0, then_norm=None):
    """out (+)= a . w^T for at most 64 rows of a, streaming w once (tensor-core kernel for decode).
    epilogue EPI_SWIGLU: w holds gate rows then (from up_row_offset) up rows; out[b, j] =
    silu(gate_j) * up_j with out [m, n], n = number of gate rows.
    `a` as NormedRows and `then_norm`: as for gemv_stream."""
    scale = a if isinstance(a, NormedRows) else None
    if scale is not None:
        a = scale.xw
    _need_cuda(a, w, out)
    if not _skinny_ok(a, w):
        raise KernelError("skinny_gemm needs bfloat16 operands, at most 64 rows, k a multiple of 8 and "
                          "16-byte aligned rows")
    m, k = a.shape
    n = out.shape[1]
    assert out.shape[0] == m and out.stride(1) == 1
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] >= up_row_offset + n
    else:
        assert w.shape[0] == n
    xw, w_next, ssq_out, cols, eps_next = _norm_producer(then_norm, epilogue, scale, m, n, -(-n // 16),
                                                         16 if m <= 16 else 64, a.device, "skinny_gemm")
    _check(_lib("fast").rllm_skinny_gemm(
        _ptr(w), _ptr(a), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(w.stride(0)),
        c_int(a.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset),
        _ptr(xw), c_int(n), _ptr(w_next), _ptr(ssq_out), *_norm_consumer(scale, epilogue, m, "skinny_gemm"), _stream()),
        "skinny_gemm")
    if then_norm is not None:
        return NormedRows(xw, ssq_out, -(-n // 16), n, eps_next, cols=cols)
    return out


def _norm_producer(then_norm, epilogue, scale, m, n, n_parts, cols, device, who):
    """Buffers of the producing side of a deferred norm: (xw, norm weight, parts, columns of a part, eps)."""
    if then_norm is None:
        return None, None, None, cols, 0.0
    if epilogue != EPI_ACCUM or scale is not None:
        raise KernelError(f"{who}: then_norm goes with the accumulate epilogue")
    w_next, eps_next = then_norm
    assert w_next.dtype == torch.float32 and w_next.numel() == n and w_next.is_contiguous()
    xw = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    ssq_out = torch.empty((max(n_parts, 1), cols), dtype=torch.float32, device=device)
    return xw, w_next, ssq_out, cols, float(eps_next)


def _norm_consumer(scale, epilogue, m, who):
    """Arguments of the consuming side of a deferred norm: parts, their number and width, d, eps."""
    if scale is None:
        return _ptr(None), c_int(0), c_int(0), c_int(0), c_float(0.0)
    if epilogue == EPI_ACCUM:
        raise KernelError(f"{who}: rows with a deferred norm go with the store and SwiGLU epilogues")
    if scale.cols < m:
        raise KernelError(f"{who}: parts of {scale.cols} columns for {m} rows")
    return _ptr(scale.ssq), c_int(scale.n_parts), c_int(scale.cols), c_int(scale.d), c_float(scale.eps)


_error_words: dict = {}
ERROR_CODES_RANGE = {4: "a token id outside the vocabulary", 5: "a cache slot outside the pool",
                     6: "a page outside the pool"}


def error_word(device) -> torch.Tensor:
    """The device int into which kernels with bounded waits write a code when a wait runs out."""
    key = torch.device(device).index or 0
    if key not in _error_words:
        _error_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_words[key]


def check_device_errors(device="cuda:0") -> None:
    """Raises if a kernel reported a fault it caught itself: a bounded wait that ran out, or an
    index that its range check refused (reads one int from the device)."""
    code = int(error_word(device).item())
    if code:
        error_word(device).zero_()
        if code in ERROR_CODES_RANGE:
            raise KernelError(f"a kernel refused an index (code {code}: {ERROR_CODES_RANGE[code]}); the access was "
                              f"skipped, the step's results are not to be used")
        raise KernelError(f"a kernel's bounded wait ran out (code {code}: 1 operand tiles never arrived, "
                          f"2 a stage was never released, 3 the accumulator never completed)")


_WAIT_LIBRARIES = {"tc": "rllm_tc", "tc2": "rllm_tc2", "stream": "rllm_stream", "attn_tc": "rllm_attn_tc"}


def set_wait_cycles(cycles: int = 0, libraries=None) -> None:
    """Limit, in clock cycles, of every bounded wait (mbarrier polls) in the kernels of the TMA
    libraries; 0 restores the default of about a second."""
    for name in (libraries or _WAIT_LIBRARIES):
        fn = getattr(_lib(name), _WAIT_LIBRARIES[name] + "_set_wait_cycles")
        fn.argtypes = [c_longlong]
        _check(fn(c_longlong(int(cycles))), f"set_wait_cycles({name})", own=False)


def wait_probe(library: str, code: int, device="cuda:0") -> None:
    """Launches the library's probe kernel: one thread waits, with the library's limit, on an
    mbarrier at which nothing arrives, gives up, writes `code` to the error word and returns."""
    fn = getattr(_lib(library), _WAIT_LIBRARIES[library] + "_wait_probe")
    with torch.cuda.device(device):
        _check(fn(_ptr(error_word(device)), c_int(code), _stream()), f"wait_probe({library})")


def _tc_ok(a, w, _meta=False) -> bool:
    """_meta: `a` stands for a freshly allocated activation (contiguous, aligned)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and (_meta or a.data_ptr() % 16 == 0) and w.data_ptr() % 16 == 0)


def gemm_tc(a, w, out, epilogue=EPI_STORE, up_row_offset=0):
    """out (+)= a . w^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory).
    epilogue as for skinny_gemm.  See gemm_tc.cu."""
    _need_cuda(a, w, out)
    if not _tc_ok(a, w):
        raise KernelError("gemm_tc needs bfloat16 operands, k a multiple of 8 and 16-byte aligned rows")
    m, k = a.shape
    n = out.shape[1]
    assert out.shape[0] == m and out.stride(1) == 1
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] >= up_row_offset + n
    else:
        assert w.shape[0] == n
    st = _lib("tc").rllm_gemm_tc(
        _ptr(a), _ptr(w), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
        c_int(w.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset),
        _ptr(error_word(a.device)), _stream())
    if st >= 30000:
        raise KernelError(f"gemm_tc: tensor map encoding failed (CUresult {st - 30000}) for m={m} n={n} k={k}")
    _check(st, "gemm_tc")
    return out


def gemm_tc2(a, w, out, epilogue=EPI_STORE, up_row_offset=0):
    """out (+)= a . w^T on the tcgen05 tensor cores with two SMs per 256 x 256 tile
    (tcgen05.mma.cta_group::2; each CTA of the pair stages half of the operands).  Arguments as
    gemm_tc.  See gemm_tc2.cu."""
    _need_cuda(a, w, out)
    if not _tc_ok(a, w):
        raise KernelError("gemm_tc2 needs bfloat16 operands, k a multiple of 8 and 16-byte aligned rows")
    m, k = a.shape
    n = out.shape[1]
    assert out.shape[0] == m and out.stride(1) == 1
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] >= up_row_offset + n
    else:
        assert w.shape[0] == n
    st = _lib("tc2").rllm_gemm_tc2(
        _ptr(a), _ptr(w), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
        c_int(w.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset),
        _ptr(error_word(a.device)), _stream())
    if st >= 30000:
        raise KernelError(f"gemm_tc2: tensor map encoding failed (CUresult {st - 30000}) for m={m} n={n} k={k}")
    _check(st, "gemm_tc2")
    return out


# From this many rows on the fused projection is at least as fast as the library product followed by the q/k
# norm + rotary kernel (us, library + kernel / fused; 8B sizes: 1,024 rows 46.6 / 46.1, 1,536 rows 64.4 / 58.2,
# 2,048 rows 90.1 / 78.1; 0.6B sizes: 512 rows 10.9 / 12.5, 1,024 rows 20.8 / 19.0; 32B sizes: 2,048 rows 170 / 147)
QKV_FUSED_MIN_ROWS = 1024
USE_QKV_FUSED = os.environ.get("RLLM_B200_NO_QKV_FUSED", "0") in ("", "0")


def can_fuse_qkv(h, w_qkv, hd: int, q_out, k_cache) -> bool:
    """Whether qkv_norm_rope_store_fused takes this step: a prompt step of many rows, bfloat16
    throughout, head size 64 or 128."""
    return (USE_QKV_FUSED and isinstance(h, torch.Tensor) and h.shape[0] >= QKV_FUSED_MIN_ROWS and hd in (64, 128)
            and _tc_ok(h, w_qkv) and q_out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and q_out.is_contiguous() and q_out.data_ptr() % 16 == 0)


def qkv_norm_rope_store_fused(h, w_qkv, q_norm_w, k_norm_w, cs_table, slots, q_out, k_cache, v_cache, H, K, hd,
                              block_size, eps, write_kv=True):
    """q_out, caches <- norm / rotary / store of h . w_qkv^T, in one kernel: the two-SM tcgen05 product
    with qk_norm_rope_store's work in its epilogue (gemm_tc2.cu); the float32 projection is never
    written.  Arguments as qk_norm_rope_store with a table of angles (or None)."""
    _need_cuda(h, w_qkv, q_out, k_cache, v_cache, slots)
    n = h.shape[0]
    if not _tc_ok(h, w_qkv) or hd not in (64, 128) or w_qkv.shape[0] != (H + 2 * K) * hd:
        raise KernelError("qkv_norm_rope_store_fused needs bfloat16 operands with 16-byte aligned rows, head size 64 "
                          "or 128 and the stacked q, k, v projections")
    assert q_out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
    assert q_out.shape == (n, H * hd) and q_out.is_contiguous() and slots.dtype == torch.int32 and slots.numel() >= n
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[-1] == hd
    if cs_table is not None:
        assert cs_table.dtype == torch.float32 and cs_table.numel() >= n * hd and cs_table.is_contiguous()
    for nw in (q_norm_w, k_norm_w):
        assert nw is None or (nw.dtype == torch.float32 and nw.numel() == hd and nw.is_contiguous())
    n_slots = k_cache.numel() // (K * hd)
    st = _lib("tc2").rllm_qkv_tc2(
        _ptr(h), _ptr(w_qkv), c_int(n), c_int(h.shape[1]), c_int(h.stride(0)), c_int(w_qkv.stride(0)), _ptr(q_out),
        _ptr(k_cache), _ptr(v_cache), _ptr(slots), _ptr(cs_table), _ptr(q_norm_w), _ptr(k_norm_w), c_int(H), c_int(K),
        c_int(hd), c_int(block_size), c_float(eps), c_int(1 if write_kv else 0), c_longlong(n_slots),
        _ptr(error_word(h.device)), _stream())
    if st >= 30000:
        raise KernelError(f"qkv_norm_rope_store_fused: tensor map encoding failed (CUresult {st - 30000})")
    _check(st, "qkv_norm_rope_store_fused")
    return q_out


def tc_swap_splits(n_tiles: int, k: int, swiglu: bool = False, n_sm: int = 148) -> int:
    """Number of K splits (CTAs of a cluster) for the swapped tcgen05 product, a power of two up to
    8 (clusters of 3, 5, 6, 7 CTAs schedule badly) that leaves every CTA at least 4 blocks of 64
    along K.  Plain products: as many as keep the CTAs under 1.6 per SM: above one per SM two CTAs
    share an SM, one streaming while the other starts or ends, and the cluster's CTAs share the
    additions and the writes.  (Measured at 24 and 64 rows on the layer sizes of Qwen3-0.6B, 8B and
    32B: 48 tiles take 4 splits, 32 take 4, 40 take 4, 8 take 8.)  SwiGLU, where the cluster's
    leader adds and writes alone: at most one CTA per SM."""
    nkb = -(-k // 64)
    if swiglu:
        limit = min(n_sm // n_tiles, nkb // 8)
    else:
        limit = min(int(1.6 * n_sm) // n_tiles, nkb // 4)
    limit = max(1, min(limit, 8))
    splits = 1
    while splits * 2 <= limit:
        splits *= 2
    return splits


def skinny_gemm_tc(a, w, out, epilogue=EPI_STORE, up_row_offset=0, n_splits=None, then_norm=None):
    """out (+)= a . w^T for at most 64 rows of a on the tcgen05 tensor cores with the weights as
    the streamed M operand (TMA ring), the K range split over the CTAs of a cluster where the weight
    matrix has few rows.  `a` as NormedRows and `then_norm`: as for gemv_stream (parts of 64 columns)."""
    scale = a if isinstance(a, NormedRows) else None
    if scale is not None:
        a = scale.xw
    _need_cuda(a, w, out)
    if not _tc_ok(a, w) or a.shape[0] > 64:
        raise KernelError("skinny_gemm_tc needs bfloat16 operands, at most 64 rows, k a multiple of 8 and "
                          "16-byte aligned rows")
    m, k = a.shape
    n = out.shape[1]
    assert out.shape[0] == m and out.stride(1) == 1
    rows_out = 64 if epilogue == EPI_SWIGLU else 128
    n_tiles = -(-n // rows_out)
    if n_splits is None:
        n_splits = tc_swap_splits(n_tiles, k, epilogue == EPI_SWIGLU, sm_count(a.device))
    n_splits = max(1, min(int(n_splits), 8))
    xw, w_next, ssq_out, cols, eps_next = _norm_producer(then_norm, epilogue, scale, m, n, n_tiles * n_splits,
                                                         TC_SWAP_NORM_COLS, a.device, "skinny_gemm_tc")
    st = _lib("tc").rllm_gemm_tc_swap(
        _ptr(w), _ptr(a), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(w.stride(0)),
        c_int(a.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset), c_int(n_splits),
        _ptr(error_word(a.device)), _ptr(xw), c_int(n), _ptr(w_next), _ptr(ssq_out),
        *_norm_consumer(scale, epilogue, m, "skinny_gemm_tc"), _stream())
    if st >= 30000:
        raise KernelError(f"skinny_gemm_tc: tensor map encoding failed (CUresult {st - 30000})")
    _check(st, "skinny_gemm_tc")
    if then_norm is not None:
        return NormedRows(xw, ssq_out, n_tiles * n_splits, n, eps_next, cols=cols)
    return out


STREAM_MAX_ROWS = 16
TC_SWAP_NORM_COLS = 64            # columns of a part of sums of squares that skinny_gemm_tc writes and reads
# a norm between two products of at most 64 rows is deferred into them (RLLM_B200_NO_DEFER_NORMS=1: never)
DEFER_NORMS = os.environ.get("RLLM_B200_NO_DEFER_NORMS", "0") in ("", "0")
_n_sm: dict = {}


def sm_count(device=None) -> int:
    """Number of SMs of the device (148 on a B200), looked up once."""
    key = torch.device(device).index if device is not None else torch.cuda.current_device()
    key = key or 0
    if key not in _n_sm:
        _n_sm[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _n_sm[key]


def stream_plan(n: int, k: int, swiglu: bool = False, n_sm: int = 148):
    """(CTAs, ring stages) of gemv_stream for n output rows: three CTAs of three stages per SM when
    each still gets three and more boxes of 8 rows, else two (measured inside the decode step of
    the 8B layer sizes: 444 x 3 for gate/up and the LM head, 296 x 3 for QKV, O and down)."""
    boxes = -(-n // 8) * (2 if swiglu else 1)
    per_sm = 3 if boxes >= 3 * 3 * n_sm else 2
    return per_sm * n_sm, 3


class NormedRows:
    """Rows of the residual stream on their way through an RMSNorm whose division has not happened
    yet: `xw` = bfloat16(x * norm weight) [m, d] and, per row, `n_parts` partial sums of squares of x
    (`ssq` [n_parts, cols] float32, row b in column b).  The product that takes them as its input
    multiplies its result rows by 1 / sqrt(sum / d + eps):  (x w r) . W^T = r ((x w) . W^T).
    Made by an accumulating launch of one of the few-row kernels (`then_norm`; gemv_stream and
    skinny_gemm up to 16 rows write parts of 16 columns, skinny_gemm above that and skinny_gemm_tc
    parts of 64), taken by `linear` and `gate_up_swiglu` in place of a tensor; each of the three
    kernels reads parts of either width."""
    __slots__ = ("xw", "ssq", "n_parts", "d", "eps", "cols")

    def __init__(self, xw, ssq, n_parts, d, eps, cols=16):
        self.xw, self.ssq, self.n_parts, self.d, self.eps, self.cols = xw, ssq, n_parts, d, eps, cols

    @property
    def shape(self):
        return self.xw.shape

    @property
    def dtype(self):
        return self.xw.dtype

    @property
    def device(self):
        return self.xw.device


def gemv_stream(a, w, out, epilogue=EPI_STORE, up_row_offset=0, grid=None, stages=None, then_norm=None):
    """out (+)= a . w^T for at most 16 rows of `a`: persistent CTAs stream their shares of w's rows
    through TMA rings (mma.sync consumers).  Epilogues as skinny_gemm.  grid, stages: number of CTAs
    and ring depth (3, 5 or 10); by default from stream_plan.
    `a` may be NormedRows (store and SwiGLU epilogues): the result rows are divided by the rows' rms.
    then_norm = (norm weight [n] float32, eps), accumulate epilogue only: the launch also prepares
    the RMSNorm of the sums it writes and returns them as NormedRows (else it returns `out`)."""
    scale = a if isinstance(a, NormedRows) else None
    if scale is not None:
        a = scale.xw
    _need_cuda(a, w, out)
    m, k = a.shape
    n = out.shape[1]
    if m > STREAM_MAX_ROWS or k % 64 or not _tc_ok(a, w):
        raise KernelError("gemv_stream: needs at most 16 rows, k % 64 == 0, bfloat16 operands with 16-byte aligned rows")
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] >= up_row_offset + n
    else:
        assert w.shape[0] == n
    assert out.stride(1) == 1 and w.shape[1] == k
    plan = stream_plan(n, k, epilogue == EPI_SWIGLU, sm_count(a.device))
    n_ctas = plan[0] if grid is None else grid
    n_parts = c_int(0)
    xw, w_next, ssq_out, cols, eps_next = _norm_producer(then_norm, epilogue, scale, m, n, n_ctas, 16, a.device,
                                                         "gemv_stream")
    st = _lib("stream").rllm_gemv_stream(
        _ptr(w), _ptr(a), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(w.stride(0)),
        c_int(a.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset),
        c_int(n_ctas), c_int(plan[1] if stages is None else stages),
        _ptr(error_word(a.device)), _ptr(xw), c_int(n), _ptr(w_next), _ptr(ssq_out), ctypes.byref(n_parts),
        *_norm_consumer(scale, epilogue, 16, "gemv_stream"), _stream())
    _check(st, "gemv_stream")
    if then_norm is not None:
        return NormedRows(xw, ssq_out, n_parts.value, n, eps_next, cols=cols)
    return out


USE_STREAM = True
STREAM_MIN_WEIGHTS = 1 << 23      # below 16 MB of weights the short-lived CTAs of skinny_gemm start faster,
STREAM_MIN_WEIGHTS_4_ROWS = 1 << 21   # but with 4 to 8 rows the norm kernels that gemv_stream saves count for more
                                  # (decode step at the 0.6B layer sizes, all four products of 4 to 12 MB on
                                  # gemv_stream against skinny_gemm: batch 1 -0.5 %, 2 -1.4 %, 4 +2.5 %, 8 +6.8 %)


def _stream_ok(a, w, _meta=False) -> bool:
    return USE_STREAM and a.shape[0] <= 8 and a.shape[1] % 64 == 0 and _tc_ok(a, w, _meta)


def _prefer_stream(a, w, n: int, swiglu: bool = False, _meta=False) -> bool:
    """gemv_stream takes up to 8 rows always, and 9 to 16 rows for the layer's plain products; with
    9 to 16 rows the gate/up product and the LM head are faster on the tcgen05 kernel (measured
    inside the decode step at batch 9, 12 and 16: 3 to 7 % of the step)."""
    m, k = a.shape
    least = STREAM_MIN_WEIGHTS_4_ROWS if 4 <= m <= 8 else STREAM_MIN_WEIGHTS
    if not USE_STREAM or k % 64 or n * k < least or not _tc_ok(a, w, _meta):
        return False
    return m <= 8 or (m <= STREAM_MAX_ROWS and not swiglu and n * k < (1 << 27))


def _prefer_tc_swap(m: int, n: int, k: int, swiglu: bool = False) -> bool:
    """Measured crossover between the two few-row kernels (B200, Qwen3-8B shapes).  The mma.sync
    kernel wins on the small per-layer matrices up to 8 rows (1.5-3 us less fixed cost); the
    tcgen05 kernel wins wherever there are more rows to multiply: everything above 16 rows, and all
    but the smallest matrix between 9 and 16 rows."""
    if k < 512 or n < 512:
        return False                      # tiny models: the fixed cost of TMEM and TMA set-up dominates
    if m <= 8:
        return False                      # (gate/up alone is 2.5 us faster on tcgen05, but not inside a decode step)
    if m <= 16:
        return n * k > 4096 * 4096
    return True


class Preceding:
    """The product launched directly before another one: its activation, its weight matrix and
    whether it was the fused gate/up product.  Handed to `linear` as `follow`, so that the second
    product takes the kernel family of the first where the shape allows it."""
    __slots__ = ("a", "w", "swiglu")

    def __init__(self, a, w, swiglu=False):
        self.a, self.w, self.swiglu = a, w, swiglu

    def took_stream(self) -> bool:
        return (self.a.dtype == torch.bfloat16
                and _prefer_stream(self.a, self.w, self.w.shape[0], swiglu=self.swiglu))


def defers_norm(m: int, w_before, w_after, swiglu_after: bool = False, w_lead=None, swiglu_lead: bool = False) -> bool:
    """Whether the RMSNorm between the accumulating product with `w_before` and the product with
    `w_after` can do without a kernel of its own at `m` rows: both products then run on one of the
    few-row kernels (gemv_stream, skinny_gemm, skinny_gemm_tc; `linear` and `gate_up_swiglu` choose
    as always), the first preparing the norm (`then_norm`), the second dividing by the rms
    (NormedRows).  The three kernels write and read the same parts of sums of squares, so any of
    them may stand on either side.  (w_lead, swiglu_lead, swiglu_after: what the caller knows of the
    products around; the answer does not depend on them.)"""
    if not DEFER_NORMS or not 0 < m <= SKINNY_MAX_ROWS:
        return False
    return all(w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[1] % 8 == 0 and w.stride(0) % 8 == 0
               and w.stride(1) == 1 and w.data_ptr() % 16 == 0 for w in (w_before, w_after))


def linear(a, w, out=None, out_dtype=None, accumulate=False, stream=None, follow=None, then_norm=None):
    """out (+)= a . w^T, choosing the kernel by element type and shape.

    float32 operands always take the plain CUDA-core product (the true 32-bit path).
    bfloat16 operands: up to 64 rows take the weight-streaming tensor-core kernel, more rows the
    library product; shapes neither can take (a row length that is not a multiple of 8
    elements) take the plain product with the same operand types."""
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        if accumulate:
            raise KernelError("linear: accumulate needs an output to add to")
        out = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    if m == 0:
        return out
    rows = a.xw if isinstance(a, NormedRows) else a          # what the rules below look at
    if rows.dtype == torch.float32 or w.dtype == torch.float32:
        if rows.dtype != w.dtype:
            raise KernelError(f"linear: activation {rows.dtype} and weight {w.dtype} differ")
        return gemm_plain(a, w, out, accumulate)
    if follow is not None and stream is None and follow.took_stream():
        stream = True
    if _skinny_ok(rows, w):
        # stream: the wish for the kernel family (a product that follows a gemv_stream launch directly
        # should be one too, whatever its size: a launch of short-lived CTAs right behind the persistent
        # ones is slow), where the shape allows it; `follow` describes the product before and decides it
        epilogue = EPI_ACCUM if accumulate else EPI_STORE
        want_stream = _prefer_stream(rows, w, n) if stream is None else (stream and _stream_ok(rows, w))
        if want_stream:
            return gemv_stream(a, w, out, epilogue, then_norm=then_norm)
        if _prefer_tc_swap(m, n, k) and out.data_ptr() % 16 == 0:
            return skinny_gemm_tc(a, w, out, epilogue, then_norm=then_norm)
        return skinny_gemm(a, w, out, epilogue, then_norm=then_norm)
    if isinstance(a, NormedRows) or then_norm is not None:
        raise KernelError("linear: a deferred norm needs a product that one of the few-row kernels takes "
                          "(ask defers_norm first)")
    aligned = (a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
               and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
               and out.stride(0) % (4 if out.dtype == torch.float32 else 8) == 0)
    if aligned:
        return gemm_lib(a, w, out, accumulate)
    return gemm_plain(a, w, out, accumulate)


def _prefer_tc2(m: int, n_col_tiles: int, n_sm: int = 148) -> bool:
    """Which of the two many-row kernels finishes the product in fewer waves: the one-CTA kernel
    walks 128-row tiles on n_sm CTAs, the two-SM kernel 256-row tiles on n_sm / 2 pairs, whose wave
    takes 0.93 of the other's (2,048 x 24,576 x 4,096: 270 us against 290 in 11 waves each).
    Measured at 12,288 x 4,096 with SwiGLU: 544 rows 116 us (two SMs) against 121, 672 rows 118
    against 128, 896 rows 160 against 141, 1,152 rows 185 against 171."""
    if not USE_TC2:
        return False
    tiles128 = -(-m // 128)
    waves_one = -(-(tiles128 * n_col_tiles) // n_sm)
    waves_two = -(-(-(-tiles128 // 2) * n_col_tiles) // (n_sm // 2))
    return 0.93 * waves_two < waves_one


USE_TC2 = True


def gate_up_swiglu(h, w_gate_up, out):
    """out[m, F] = silu(h . Wg^T) * (h . Wu^T) with w_gate_up = [Wg; Wu] stacked ([2F, k]).
    bfloat16: one kernel (the weight-streaming kernel up to 64 rows, the tcgen05 kernel above);
    float32 and odd shapes: a product followed by the activation kernel."""
    m = h.shape[0]
    F = out.shape[1]
    rows = h.xw if isinstance(h, NormedRows) else h
    if _skinny_ok(rows, w_gate_up):
        if _prefer_stream(rows, w_gate_up, 2 * F, swiglu=True):
            return gemv_stream(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F)
        if _prefer_tc_swap(m, 2 * F, h.shape[1], swiglu=True):
            return skinny_gemm_tc(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F)
        return skinny_gemm(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F)
    if isinstance(h, NormedRows):
        raise KernelError("gate_up_swiglu: a deferred norm needs a product that one of the few-row kernels takes")
    if _tc_ok(h, w_gate_up) and out.data_ptr() % 16 == 0:
        # tcgen05, activation in the epilogue; two SMs per tile where that takes fewer waves
        many = gemm_tc2 if _prefer_tc2(m, -(-F // 128), sm_count(h.device)) else gemm_tc
        return many(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F)
    gu = linear(h, w_gate_up, out_dtype=torch.float32)     # same rounding points as the fused kernels
    return silu_mul(gu, out)


FLASH_HEAD_DIMS = (64, 128)
USE_ATTENTION_TC = True        # prompt portions with head size 128 take the tcgen05 kernel where it applies
DECODE_SPLIT_KEYS = 128        # keys per split of the decode shape: a constant, so that a request's
                               # result never depends on the batch around it
DECODE_MAX_Q = 8               # requests with at most this many tokens in the step take the decode shape
DECODE_ROWS = 8                # (token, head) rows of a decode tile: 8 takes the kernel with the keys as the M side


class AttentionPlan:
    """Tiles of one step for one attention geometry (query heads per key/value head, window):
    which requests take the decode shape (16-row tiles, split keys) and which the prefill shape
    (64-row tiles).  Built once per step on the host and shared by every layer of that geometry."""

    def __init__(self, ctx, H, K, window, device):
        g = H // K
        self.GHd = min(g, DECODE_ROWS)
        self.chunks_d = -(-g // self.GHd)
        self.GHp = min(g, 64)
        self.chunks_p = -(-g // self.GHp)
        self.TTp = 64 // self.GHp
        dec = [r for r in range(ctx.n_requests) if ctx.q_lens[r] <= DECODE_MAX_Q]
        pre = [r for r in range(ctx.n_requests) if ctx.q_lens[r] > DECODE_MAX_Q]
        self.TTd = 1 if all(ctx.q_lens[r] == 1 for r in dec) else max(1, DECODE_ROWS // self.GHd)
        cu = [0]
        for ql in ctx.q_lens:
            cu.append(cu[-1] + ql)
        d_req, d_tok, p_req, p_tok = [], [], [], []
        n_splits = 1
        for r in dec:
            for t0 in range(0, ctx.q_lens[r], self.TTd):
                d_req.append(r)
                d_tok.append(cu[r] + t0)
                pos_first = ctx.start_pos[r] + t0
                pos_last = ctx.start_pos[r] + min(t0 + self.TTd, ctx.q_lens[r]) - 1
                # an upper bound of the keys the tile reads (the kernel rounds the window's start
                # down to a multiple of 32); a function of the padded shape only, so that a graph
                # captured for a padded context covers every real one
                span = pos_last + 1
                if window > 0:
                    span = min(span, window + self.TTd + 30)
                n_splits = max(n_splits, -(-span // DECODE_SPLIT_KEYS))
        for r in pre:
            for t0 in range(0, ctx.q_lens[r], self.TTp):
                p_req.append(r)
                p_tok.append(cu[r] + t0)
        # tiles of the tcgen05 kernel: 128 rows = (128 / g) tokens x g heads, when g divides 128
        t_req, t_tok = [], []
        self.TTt = 128 // g if g <= 128 and 128 % g == 0 else 0
        if self.TTt:
            for r in pre:
                for t0 in range(0, ctx.q_lens[r], self.TTt):
                    t_req.append(r)
                    t_tok.append(cu[r] + t0)
        self.n_dec, self.n_pre, self.n_tc, self.n_splits = len(d_req), len(p_req), len(t_req), n_splits
        flat = torch.tensor(d_req + d_tok + p_req + p_tok + t_req + t_tok + [0], dtype=torch.int32).to(device)
        nd, np_, nt = self.n_dec, self.n_pre, self.n_tc
        self.d_req, self.d_tok = flat[:nd], flat[nd:2 * nd]
        self.p_req, self.p_tok = flat[2 * nd:2 * nd + np_], flat[2 * nd + np_:2 * nd + 2 * np_]
        o = 2 * nd + 2 * np_
        self.t_req, self.t_tok = flat[o:o + nt], flat[o + nt:o + 2 * nt]


def paged_flash_attention(q, k_cache, v_cache, out, positions, cu_q, block_table, tile_req, tile_tok0,
                          n_tiles, H, K, hd, block_size, scale, window, mode, TT, GH, head_chunks,
                          split_keys=DECODE_SPLIT_KEYS, n_splits=1):
    """Tensor-core paged attention; mode 0: prefill shape, mode 1: decode shape with split keys
    (allocates the partials as scratch).  See attention_flash.cu."""
    _need_cuda(q, k_cache, v_cache, out, positions, cu_q, block_table, tile_req, tile_tok0)
    _need_contig(q=q, k_cache=k_cache, v_cache=v_cache, out=out)
    if q.dtype != torch.bfloat16 or hd not in FLASH_HEAD_DIMS:
        raise KernelError(f"paged_flash_attention takes bfloat16 and a head size of 64 or 128, got {q.dtype}, {hd}")
    assert block_table.stride(1) == 1
    part_o = part_ml = None
    if mode == 1:
        rows = n_tiles * K * head_chunks * n_splits * TT * GH
        part_o = torch.empty(rows * hd, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(rows * 2, dtype=torch.float32, device=q.device)
    _check(_lib("attn").rllm_paged_flash_attention(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(positions),
        _ptr(cu_q), _ptr(block_table), c_int(block_table.stride(0)), _ptr(tile_req), _ptr(tile_tok0),
        c_int(n_tiles), c_int(H), c_int(K), c_int(hd), c_int(block_size), c_float(scale), c_int(window),
        c_int(mode), c_int(TT), c_int(GH), c_int(head_chunks), c_int(split_keys), c_int(n_splits),
        c_longlong(k_cache.shape[0]), _ptr(error_word(q.device)), _stream()), "paged_flash_attention")
    global _launches
    if mode == 1:
        _launches += 1                         # the combine kernel
    return out


def attention_tc_ok(q, hd, block_size, H, K) -> bool:
    g = H // K
    return (q.dtype == torch.bfloat16 and hd == 128 and 8 <= block_size <= 128
            and block_size & (block_size - 1) == 0 and g <= 128 and 128 % g == 0)


def attention_tc(q, k_cache, v_cache, out, positions, cu_q, block_table, tile_req, tile_tok0, n_tiles, H, K, hd,
                 block_size, scale, window):
    """Prefill attention on the tcgen05 tensor cores (S and O in tensor memory); see attention_tc.cu."""
    _need_cuda(q, k_cache, v_cache, out, positions, cu_q, block_table, tile_req, tile_tok0)
    _need_contig(q=q, k_cache=k_cache, v_cache=v_cache, out=out)
    if not attention_tc_ok(q, hd, block_size, H, K):
        raise KernelError("attention_tc takes bfloat16, head size 128, a power-of-two page size from 8 to 128 and "
                          "a number of query heads per key/value head that divides 128")
    st = _lib("attn_tc").rllm_attention_tc(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), c_int(q.shape[0]), c_longlong(k_cache.shape[0]),
        _ptr(positions), _ptr(cu_q), _ptr(block_table), c_int(block_table.stride(0)), _ptr(tile_req),
        _ptr(tile_tok0), c_int(n_tiles), c_int(H), c_int(K), c_int(hd), c_int(block_size), c_float(scale),
        c_int(window), _ptr(error_word(q.device)), _stream())
    if st >= 30000:
        raise KernelError(f"attention_tc: tensor map encoding failed (CUresult {st - 30000})")
    _check(st, "attention_tc")
    return out


def paged_attention(q, k_cache, v_cache, out, ctx, block_table, H, K, hd, block_size, scale, window=0):
    """Attention of the step's tokens over the paged cache; chooses the kernel by element type,
    head size and the shape of the step (`ctx`: the step's StepContext).  float32, and head sizes
    other than 64 and 128, take the plain kernel."""
    if q.dtype != torch.bfloat16 or hd not in FLASH_HEAD_DIMS:
        return paged_attention_generic(q, k_cache, v_cache, out, ctx.positions, ctx.seq_ids, block_table,
                                       H, K, hd, block_size, scale, window)
    key = (H // K, window)
    plan = ctx.plans.get(key)
    if plan is None:
        plan = ctx.plans[key] = AttentionPlan(ctx, H, K, window, q.device)
    if plan.n_pre and plan.n_tc and USE_ATTENTION_TC and attention_tc_ok(q, hd, block_size, H, K):
        attention_tc(q, k_cache, v_cache, out, ctx.positions, ctx.cu_q, block_table, plan.t_req, plan.t_tok,
                     plan.n_tc, H, K, hd, block_size, scale, window)
    elif plan.n_pre:
        paged_flash_attention(q, k_cache, v_cache, out, ctx.positions, ctx.cu_q, block_table, plan.p_req,
                              plan.p_tok, plan.n_pre, H, K, hd, block_size, scale, window, 0, plan.TTp,
                              plan.GHp, plan.chunks_p)
    if plan.n_dec:
        paged_flash_attention(q, k_cache, v_cache, out, ctx.positions, ctx.cu_q, block_table, plan.d_req,
                              plan.d_tok, plan.n_dec, H, K, hd, block_size, scale, window, 1, plan.TTd,
                              plan.GHd, plan.chunks_d, DECODE_SPLIT_KEYS, plan.n_splits)
    return out
