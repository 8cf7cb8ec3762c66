"""Loads a model's tensors by name from ``model.safetensors``, or from the shards that a
``model.safetensors.index.json`` weight map names, and checks them against what the model's
parts expect.  One error lists every missing tensor, every unexpected tensor and every
wrong shape at once.

Element types: floating-point tensors stored in 16 bits are kept as bfloat16 (float16 is
converted), tensors stored in 32 bits stay 32-bit, integer tensors become int32.  What a part
does with its tensors afterwards (concatenating projections, converting norm weights to
float32) is that part's load-time transform.

AxiomOperator/rllm loads by name in the same way, one ``require_tensor`` per weight
(crates/rllm-model/src/loader.rs:8-23, crates/rllm-model/src/qwen3.rs:124-160).
"""
from __future__ import annotations

import json
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


INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"


def weight_files(model_dir) -> tuple[dict, list]:
    """Which file holds which tensor.  A folder holds either ``model.safetensors`` or a weight map
    ``model.safetensors.index.json`` (``{"weight_map": {tensor name: file name}}``) beside the
    shards it names (``model-00001-of-0000N.safetensors`` and so on).  Returns (name -> path from
    the index, or {} for a single file; the list of files to open).  Errors name the file."""
    model_dir = Path(model_dir)
    index = model_dir / INDEX_NAME
    single = model_dir / SINGLE_NAME
    if not index.is_file():
        if not single.is_file():
            raise WeightFileError(f"{model_dir}: neither {SINGLE_NAME} nor {INDEX_NAME} is there")
        return {}, [single]
    try:
        doc = json.loads(index.read_text())
        wmap = doc["weight_map"]
        if not isinstance(wmap, dict) or not wmap:
            raise TypeError
    except (json.JSONDecodeError, UnicodeDecodeError, KeyError, TypeError):
        raise WeightFileError(f"{index}: not a weight map ({{\"weight_map\": {{tensor: file}}}} expected)") from None
    where = {}
    for name, fname in wmap.items():
        if not isinstance(fname, str) or "/" in fname or "\\" in fname or fname in ("", ".", ".."):
            raise WeightFileError(f"{index}: tensor {name!r} is mapped to {fname!r}, which is not a file name in this folder")
        where[name] = model_dir / fname
    files = sorted(set(where.values()))
    for path in files:
        if not path.is_file():
            names = [n for n, q in where.items() if q == path]
            raise WeightFileError(f"{path}: the shard is missing ({index.name} puts {len(names)} tensors there, "
                                  f"e.g. {names[0]})")
    return where, files


def load_checked(model_dir, expected: Mapping[str, tuple], ignorable: Iterable[str] = ()) -> dict:
    """Reads the folder's weights: ``model.safetensors``, or every shard that
    ``model.safetensors.index.json`` names.  `expected` maps tensor name -> shape; names in
    `ignorable` may be present without being used (e.g. an lm_head stored beside tied
    embeddings).  Returns name -> CPU tensor (a view of the file's memory map) for the expected
    names.  One WeightMismatchError lists missing, unexpected and wrong-shaped tensors of all files
    together; a shard that is missing, a tensor that is not in the shard the index names and a
    tensor stored in two shards are WeightFileErrors that name the file."""
    model_dir = Path(model_dir)
    ignorable = set(ignorable)
    where, files = weight_files(model_dir)
    opened = {}
    try:
        for path in files:
            opened[path] = SafetensorsFile(path)
        home = {}                                    # tensor name -> the file that stores it
        for path, f in opened.items():
            for n in f.names():
                if n in home:
                    raise WeightFileError(f"{path}: tensor {n!r} is stored here and in {home[n].name}")
                home[n] = path
        for n, path in where.items():
            if home.get(n) != path:
                also = f" (it is in {home[n].name})" if n in home else ""
                raise WeightFileError(f"{path}: {INDEX_NAME} puts tensor {n!r} here, but the file does not hold it{also}")
        shown = model_dir / (INDEX_NAME if where else SINGLE_NAME)
        missing = sorted(n for n in expected if n not in home)
        unexpected = sorted(n for n in home if n not in expected and n not in ignorable)
        wrong = sorted((n, opened[home[n]].shape(n), tuple(expected[n])) for n in expected
                       if n in home and opened[home[n]].shape(n) != tuple(expected[n]))
        if missing or unexpected or wrong:
            raise WeightMismatchError(shown, missing, unexpected, wrong)
        return {n: normalize_dtype(opened[home[n]].tensor(n)) for n in expected}
    finally:
        for f in opened.values():
            f.close()
