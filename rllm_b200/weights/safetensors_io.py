"""Reader and writer for the safetensors file format (8-byte little-endian header length, a
JSON header ``{name: {dtype, shape, data_offsets}}``, then the raw little-endian tensor data).

Tensors come back as CPU torch tensors over a memory map of the file (no copy until they
are moved to the device).  The header is checked before anything is touched: length,
JSON, known element types, offsets inside the file, byte counts that match the shapes, and
no overlap.  AxiomOperator/rllm does the same checks on its GGUF index
(crates/rllm-gguf/src/lib.rs:169-240) and hands out zero-copy views of the map
(crates/rllm-model/src/loader.rs:8-23).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import numpy as np
import torch


class WeightFileError(ValueError):
    """A weight file that cannot be read; the message names the file and the tensor."""


# safetensors dtype -> (numpy carrier type, torch type, bytes per element)
_DTYPES = {
    "F32": (np.float32, torch.float32, 4),
    "F16": (np.float16, torch.float16, 2),
    "BF16": (np.uint16, torch.bfloat16, 2),
    "F64": (np.float64, torch.float64, 8),
    "I64": (np.int64, torch.int64, 8),
    "I32": (np.int32, torch.int32, 4),
    "I16": (np.int16, torch.int16, 2),
    "I8": (np.int8, torch.int8, 1),
    "U8": (np.uint8, torch.uint8, 1),
    "BOOL": (np.bool_, torch.bool, 1),
}
_TORCH_TO_ST = {v[1]: k for k, v in _DTYPES.items()}
MAX_HEADER_BYTES = 100 * 1024 * 1024


def read_header(path) -> tuple[dict, int, int]:
    """Returns (header without __metadata__, offset of the data section, file size) after checking it."""
    path = Path(path)
    if not path.is_file():
        raise WeightFileError(f"{path}: no such file")
    size = path.stat().st_size
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise WeightFileError(f"{path}: truncated (no header length)")
        (hlen,) = struct.unpack("<Q", head)
        if hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise WeightFileError(f"{path}: header length {hlen} is larger than the file or the limit "
                                  f"of {MAX_HEADER_BYTES} bytes")
        raw = f.read(hlen)
    try:
        header = json.loads(raw)
    except (json.JSONDecodeError, UnicodeDecodeError) as e:
        raise WeightFileError(f"{path}: header is not valid JSON ({e})") from None
    if not isinstance(header, dict):
        raise WeightFileError(f"{path}: header must be a JSON object")
    header.pop("__metadata__", None)
    base = 8 + hlen
    spans = []
    for name, info in header.items():
        if not isinstance(info, dict) or not {"dtype", "shape", "data_offsets"} <= set(info):
            raise WeightFileError(f"{path}: tensor {name!r}: entry needs dtype, shape and data_offsets")
        if info["dtype"] not in _DTYPES:
            raise WeightFileError(f"{path}: tensor {name!r}: element type {info['dtype']!r} is not supported")
        shape = info["shape"]
        if not isinstance(shape, list) or any((not isinstance(s, int)) or s < 0 for s in shape):
            raise WeightFileError(f"{path}: tensor {name!r}: bad shape {shape!r}")
        try:
            lo, hi = info["data_offsets"]
        except (TypeError, ValueError):
            raise WeightFileError(f"{path}: tensor {name!r}: bad data_offsets") from None
        count = 1
        for s in shape:
            count *= s
        nbytes = count * _DTYPES[info["dtype"]][2]
        if not (isinstance(lo, int) and isinstance(hi, int)) or lo < 0 or hi < lo or hi - lo != nbytes:
            raise WeightFileError(f"{path}: tensor {name!r}: data_offsets {info['data_offsets']!r} do not "
                                  f"hold {nbytes} bytes for shape {shape} of {info['dtype']}")
        if base + hi > size:
            raise WeightFileError(f"{path}: tensor {name!r}: data ends at byte {base + hi} but the file "
                                  f"has {size} (truncated file)")
        if hi > lo:
            spans.append((lo, hi, name))
    spans.sort()
    for (lo0, hi0, n0), (lo1, hi1, n1) in zip(spans, spans[1:]):
        if lo1 < hi0:
            raise WeightFileError(f"{path}: tensors {n0!r} and {n1!r} overlap in the data section")
    return header, base, size


class SafetensorsFile:
    """A memory-mapped safetensors file: ``names()``, ``shape(name)``, ``dtype(name)``, ``tensor(name)``."""

    def __init__(self, path):
        self.path = Path(path)
        self.header, self._base, size = read_header(self.path)
        self._file = open(self.path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return list(self.header)

    def shape(self, name):
        return tuple(self.header[name]["shape"])

    def dtype(self, name) -> torch.dtype:
        return _DTYPES[self.header[name]["dtype"]][1]

    def tensor(self, name) -> torch.Tensor:
        info = self.header[name]
        np_t, torch_t, _ = _DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        count = (hi - lo) // _DTYPES[info["dtype"]][2]
        if count == 0:
            return torch.empty(info["shape"], dtype=torch_t)
        arr = np.frombuffer(self._map, dtype=np_t, count=count, offset=self._base + lo)
        # the map is read-only; torch warns about non-writable arrays, so take a private copy lazily:
        # tensors are moved to the device right after, the copy is what that move reads.
        t = torch.from_numpy(arr.copy())
        if torch_t == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(info["shape"])

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Writes `tensors` (name -> CPU torch tensor) in name order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise WeightFileError(f"tensor {name!r}: element type {t.dtype} cannot be written")
        if t.dtype == torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
