"""One registry from an architecture's name (config.json ``architectures[0]``) to its typed
configuration class; the configuration in turn describes the model.  AxiomOperator/rllm keeps
the same single switch in ``AnyModel::load`` (crates/rllm-model/src/lib.rs:204-212)."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Type

from .base import ConfigError, ModelConfig

_ARCHITECTURES: dict[str, Type[ModelConfig]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig]) -> Type[ModelConfig]:
    """Registers `config_cls` under `name`.  Registering a name twice replaces the entry."""
    _ARCHITECTURES[name] = config_cls
    return config_cls


def supported_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class(name: str) -> Type[ModelConfig]:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unsupported architecture {name!r} (supported: "
                          f"{', '.join(supported_architectures())})") from None


def config_from_dict(d: Mapping[str, Any]) -> ModelConfig:
    archs = d.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: required key 'architectures' is missing or not a list of names")
    return config_class(archs[0]).from_dict(d)


def load_config(model_dir) -> ModelConfig:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no such file")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)
