"""Loads a model's tensors by name from ``model.safetensors`` and checks them against what the
model's parts expect.  One error lists every missing tensor, every unexpected tensor and every
wrong shape at once.

Element types: floating-point tensors stored in 16 bits are kept as bfloat16 (float16 is
converted), tensors stored in 32 bits stay 32-bit, integer tensors become int32.  What a part
does with its tensors afterwards (concatenating projections, converting norm weights to
float32) is that part's load-time transform.

AxiomOperator/rllm loads by name in the same way, one ``require_tensor`` per weight
(crates/rllm-model/src/loader.rs:8-23, crates/rllm-model/src/qwen3.rs:124-160).
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterable, Mapping

import torch

from .safetensors_io import SafetensorsFile, WeightFileError


class WeightMismatchError(ValueError):
    """The file's tensors do not match the model; carries the three lists."""

    def __init__(self, path, missing, unexpected, wrong_shape):
        self.path, self.missing, self.unexpected, self.wrong_shape = path, missing, unexpected, wrong_shape
        lines = [f"{path}: the file's tensors do not match the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        super().__init__("\n".join(lines))


def normalize_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.float32, torch.bfloat16, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if not t.dtype.is_floating_point:
        return t.to(torch.int32)
    return t.to(torch.bfloat16)


def load_checked(model_dir, expected: Mapping[str, tuple], ignorable: Iterable[str] = ()) -> dict:
    """Reads ``model_dir/model.safetensors``.  `expected` maps tensor name -> shape; names in
    `ignorable` may be present without being used (e.g. an lm_head stored beside tied
    embeddings).  Returns name -> CPU tensor for the expected names."""
    path = Path(model_dir) / "model.safetensors"
    ignorable = set(ignorable)
    with SafetensorsFile(path) as f:
        have = set(f.names())
        missing = sorted(n for n in expected if n not in have)
        unexpected = sorted(n for n in have if n not in expected and n not in ignorable)
        wrong = sorted((n, f.shape(n), tuple(expected[n])) for n in expected
                       if n in have and f.shape(n) != tuple(expected[n]))
        if missing or unexpected or wrong:
            raise WeightMismatchError(path, missing, unexpected, wrong)
        return {n: normalize_dtype(f.tensor(n)) for n in expected}
