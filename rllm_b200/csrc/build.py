"""Builds the CUDA libraries of this package for sm_100a with nvcc and loads them with ctypes.

Each library is a group of ``.cu`` files compiled to one shared object with plain
``extern "C"`` entry points (no Python or torch headers, so a file compiles in
seconds).  A library is built the first time something asks for it and is rebuilt
when one of its sources, a header or the flags change (content hash beside the
object).  Objects go to ``_build/`` next to the sources, or, when that folder cannot
be written, to ``$RLLM_B200_BUILD_DIR`` or a per-user folder under the system's
temporary directory.  Nothing here needs a GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]

# library name -> (sources, extra link flags)
LIBRARIES = {
    "core": (["elementwise.cu", "attention_generic.cu", "gemm_plain.cu", "sampling.cu"], []),
    "blas": (["gemm_lib.cu"], ["-lcublas"]),
    "fast": (["skinny_gemm.cu"], []),
    "attn": (["attention_flash.cu"], []),
    "tc": (["gemm_tc.cu"], []),
    "tc2": (["gemm_tc2.cu"], []),
    "stream": (["gemv_stream.cu"], []),
    "attn_tc": (["attention_tc.cu"], []),
    "host": (["host_runtime.cpp"], []),
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("RLLM_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BuildError("nvcc not found (looked at $RLLM_B200_NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels of rllm_b200 cannot be built")


def build_dir() -> Path:
    """The first writable folder of: $RLLM_B200_BUILD_DIR, csrc/_build, <tmp>/rllm_b200_build_<uid>."""
    cands = []
    if os.environ.get("RLLM_B200_BUILD_DIR"):
        cands.append(Path(os.environ["RLLM_B200_BUILD_DIR"]))
    cands.append(CSRC / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"rllm_b200_build_{os.getuid()}")
    for c in cands:
        try:
            c.mkdir(parents=True, exist_ok=True)
            probe = c / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return c
        except OSError:
            continue
    raise BuildError("no writable build folder among: " + ", ".join(map(str, cands)))


def _digest(paths, flags) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:20]


def _say(msg: str) -> None:
    print(f"[rllm_b200 build] {msg}", file=sys.stderr, flush=True)


def _run(cmd, what):
    """Runs a compiler command; prints a line every few seconds while it runs."""
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def tick():
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")
    th = threading.Thread(target=tick, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"{what} failed (exit {proc.returncode}):\n{' '.join(map(str, cmd))}\n{out}")
    return out


def library_path(name: str) -> Path:
    return build_dir() / f"librllm_{name}.so"


def build(name: str, verbose: bool = True) -> Path:
    """Compiles library `name` if it is missing or stale; returns the path of the shared object."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r} (known: {sorted(LIBRARIES)})")
    sources, link_flags = LIBRARIES[name]
    srcs = [CSRC / s for s in sources]
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    flags = NVCC_FLAGS + link_flags
    out_dir = build_dir()
    so = out_dir / f"librllm_{name}.so"
    stamp = out_dir / f"librllm_{name}.stamp"
    want = _digest(srcs + headers, flags)
    if so.exists() and stamp.exists() and stamp.read_text().strip() == want:
        return so
    if all(p.suffix == ".cpp" for p in srcs):
        # host-only library: the C++ compiler alone
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler (g++) found for the host runtime")
        tmp_so = out_dir / f".librllm_{name}.{os.getpid()}.so"
        _run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-o", str(tmp_so), *map(str, srcs)], f"{name} (host C++)")
        os.replace(tmp_so, so)
        stamp.write_text(want)
        return so
    nvcc = _nvcc()
    if verbose:
        _say(f"compiling library '{name}' ({len(srcs)} files) for sm_100a into {out_dir}")
    t0 = time.time()
    hdr_digest = _digest(headers, NVCC_FLAGS)

    def compile_one(src: Path) -> Path:
        obj = out_dir / f"{name}_{src.stem}.o"
        ostamp = out_dir / f"{name}_{src.stem}.ostamp"
        w = _digest([src], NVCC_FLAGS) + hdr_digest
        if obj.exists() and ostamp.exists() and ostamp.read_text().strip() == w:
            return obj
        _run([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], src.name)
        ostamp.write_text(w)
        if verbose:
            _say(f"compiled {src.name} ({time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp_so = out_dir / f".librllm_{name}.{os.getpid()}.so"
    _run([nvcc, "-shared", "--cudart", "shared", "-o", str(tmp_so), *map(str, objs), *link_flags], f"link {so.name}")
    os.replace(tmp_so, so)
    stamp.write_text(want)
    if verbose:
        _say(f"library '{name}' ready ({time.time() - t0:.0f} s)")
    return so


def load(name: str) -> ctypes.CDLL:
    """Builds (if needed) and loads library `name`.  Raises BuildError when it cannot: there is
    no fallback path without the compiled kernels."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            so = build(name)
            try:
                lib = ctypes.CDLL(str(so))
            except OSError as e:
                raise BuildError(f"cannot load {so}: {e}") from e
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> list[Path]:
    return [build(n, verbose) for n in LIBRARIES]
