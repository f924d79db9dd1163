"""Typed model configuration: the base class and the config.json reader.

A configuration is a frozen dataclass whose fields are the architecture's own
config.json keys.  Every size and constant the model code uses comes from one of
these fields; the model code holds no literals of its own.  (The reference keeps
every size as a literal in its model program, src/models/gpt2_small.sandy.go:7,18,36,52;
here they are data.)
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, ClassVar, Dict


class ConfigError(ValueError):
    """A config.json that is missing, malformed or names impossible sizes."""


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's typed configuration."""

    # Name under which the architecture is registered ("GPT2LMHeadModel", ...).
    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def validate(self) -> None:
        raise NotImplementedError


def _require(raw: Dict[str, Any], key: str, kind, *, default=dataclasses.MISSING):
    """Fetch `key` from a parsed config.json with a type check and a clear error."""
    if key not in raw or raw[key] is None:
        if default is dataclasses.MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    value = raw[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if kind is int and isinstance(value, bool):
        raise ConfigError(f"config.json: key '{key}' must be an integer, got {value!r}")
    if not isinstance(value, kind):
        raise ConfigError(
            f"config.json: key '{key}' must be {kind.__name__}, got {type(value).__name__} {value!r}")
    return value


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder '{model_dir}'")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw


def architecture_name(raw: Dict[str, Any]) -> str:
    """The registry key of a parsed config.json: `architectures[0]`."""
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]


def load_config(model_dir: str) -> ModelConfig:
    """Read `model_dir/config.json` and return the typed configuration of the
    architecture it names.  The class is chosen by the registry, never by the caller."""
    from ..registry import get_architecture

    raw = read_config_json(model_dir)
    arch = get_architecture(architecture_name(raw))
    cfg = arch.config_cls.from_dict(raw)
    cfg.validate()
    return cfg


def save_config(cfg: ModelConfig, model_dir: str) -> str:
    os.makedirs(model_dir, exist_ok=True)
    path = os.path.join(model_dir, "config.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(cfg.to_dict(), f, indent=2, sort_keys=True)
        f.write("\n")
    return path
