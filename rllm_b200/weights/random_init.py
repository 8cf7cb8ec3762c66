"""Random-weights mode: makes a model folder (config.json, model.safetensors) from a typed
configuration and a seed.  Matrices are N(0, std), norm weights 1 + N(0, norm_std); every tensor
has its own generator seeded from (seed, tensor name), so a tensor's values do not depend on
which other tensors the model has.  AxiomOperator/rllm has no such feature; its tests
synthesize tensors the same way (crates/rllm-cuda/tests/common/parity.rs:41-96).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from ..config.base import ModelConfig
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(h[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensors(expected: dict, seed: int, dtype=torch.bfloat16, std=0.02, norm_std=0.1,
                   device="cpu") -> dict:
    """`expected`: name -> (shape, role) with role 'norm' (1 + noise) or anything else (noise)."""
    out = {}
    for name, (shape, role) in expected.items():
        g = _generator(seed, name, device)
        t = torch.randn(shape, generator=g, dtype=torch.float32, device=device)
        t = 1.0 + norm_std * t if role == "norm" else std * t
        out[name] = t.to(dtype)
    return out


def write_random_model(config: ModelConfig, out_dir, seed: int = 0, dtype=torch.bfloat16,
                       std: float = 0.02, norm_std: float = 0.1, shards: int = 1) -> Path:
    """Writes `out_dir/config.json` and `out_dir/model.safetensors`; returns `out_dir`.
    With shards > 1 the tensors (the same values) go, in name order and in runs of about equal
    bytes, into ``model-0000i-of-0000N.safetensors`` beside a ``model.safetensors.index.json``
    weight map, the layout in which large checkpoints are stored."""
    from ..models.model import expected_tensors     # late: models imports weights
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[dtype]
    (out_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    tensors = random_tensors(expected_tensors(config.model_spec()), seed, dtype, std, norm_std)
    meta = {"format": "pt", "seed": seed}
    if shards <= 1:
        write_safetensors(out_dir / "model.safetensors", tensors, meta)
        return out_dir
    write_sharded(out_dir, tensors, shards, meta)
    return out_dir


def write_sharded(out_dir, tensors: dict, shards: int, metadata: dict | None = None) -> list:
    """Writes `tensors` as `shards` files and their weight map; returns the files' names."""
    out_dir = Path(out_dir)
    names = sorted(tensors)
    shards = max(1, min(int(shards), len(names)))
    total = sum(tensors[n].numel() * tensors[n].element_size() for n in names)
    groups, acc = [[] for _ in range(shards)], 0
    for i, n in enumerate(names):
        # the shard whose byte range the tensor starts in, but never so far ahead that a later shard stays empty
        g = min(acc * shards // max(total, 1), i, shards - 1)
        g = max(g, shards - (len(names) - i))
        groups[g].append(n)
        acc += tensors[n].numel() * tensors[n].element_size()
    files, wmap = [], {}
    for g, members in enumerate(groups):
        fname = f"model-{g + 1:05d}-of-{shards:05d}.safetensors"
        write_safetensors(out_dir / fname, {n: tensors[n] for n in members}, metadata)
        files.append(fname)
        wmap.update({n: fname for n in members})
    (out_dir / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {"total_size": total}, "weight_map": wmap}, indent=1))
    return files
