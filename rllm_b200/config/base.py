"""Typed model configuration and the description of a model as data.

A configuration class reads the architecture's own config.json keys
(``from_dict``) and turns itself into a :class:`ModelSpec`: a list of layers, each
put together from named parts with their sizes and constants as parameters, and
the order in which the layers run.  Nothing below this file knows an
architecture's name; code never holds a size or a constant that config.json gives.

AxiomOperator/rllm keeps the same split: a typed ``Qwen3Config``
(crates/rllm-model/src/qwen3.rs:17-96) and parts that take their constants as
arguments (crates/rllm-core/src/lib.rs:264-279, 412-413).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered kind, its parameters, and the prefix its tensors
    carry in the weight file (e.g. ``model.layers.3.self_attn.``)."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """A layer: how its parts are arranged (`block`) and the parts themselves.  `position` is
    the position encoding handed to the mixer (None: the mixer uses none)."""
    block: str
    mixer: PartSpec
    ffn: PartSpec
    norms: Mapping[str, PartSpec]
    position: Optional[PartSpec] = None


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: which layer runs, and whose cache its mixer uses.
    `cache_of` is the index of an EARLIER run entry whose cache this one reads without
    writing (None: the entry owns a cache of its own and writes it)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder as data."""
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: tuple            # of LayerSpec
    run_order: tuple         # of RunEntry; may name a layer twice
    final_norm: PartSpec
    lm_head: PartSpec
    max_position: int


def require(d: Mapping[str, Any], key: str, typ, where: str = "config.json"):
    if key not in d or d[key] is None:
        raise ConfigError(f"{where}: required key '{key}' is missing")
    return coerce(d[key], key, typ, where)


def optional(d: Mapping[str, Any], key: str, typ, default, where: str = "config.json"):
    if key not in d or d[key] is None:
        return default
    return coerce(d[key], key, typ, where)


def coerce(v, key, typ, where="config.json"):
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"{where}: key '{key}' must be an integer, got {v!r}")
        return int(v)
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: key '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"{where}: key '{key}' must be true or false, got {v!r}")
        return v
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"{where}: key '{key}' must be a string, got {v!r}")
        return v
    return v


class ModelConfig:
    """Base of the typed configurations.  Subclasses are dataclasses with

    * ``architecture``: the name under which they register,
    * ``from_dict(d)``: parse and validate config.json's keys,
    * ``to_dict()``: the config.json keys again (the random-weights mode writes them),
    * ``model_spec()``: the model as data.
    """
    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError
