"""Typed model configuration: the base class and the config.json reader.

A configuration is a typed object whose fields are the architecture's own config.json keys.  Every
size and constant the model code uses comes from one of these fields; the model code holds no
literals of its own.  (The reference keeps every size as a literal in its model program,
src/models/gpt2_small.sandy.go:7,18,36,52; here they are data.)

Reading, type checks and validation are the host library's (core/config.cpp); the classes here are
its typed results on the Python side.  An architecture defined in Python subclasses ModelConfig and
registers itself (registry.register_architecture); the library then calls its `from_dict`,
`validate` and `describe` through callbacks.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict

from .. import core
from ..errors import ConfigError  # noqa: F401  (re-exported)


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


def architecture_name(raw: Dict[str, Any]) -> str:
    """The registry key of a parsed config.json: `architectures[0]`."""
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]


def config_from_normalised(normalised: Dict[str, Any]) -> ModelConfig:
    """The typed Python object for a configuration the library has read and checked."""
    from ..registry import get_architecture

    arch = get_architecture(architecture_name(normalised))
    return arch.config_cls.from_dict(normalised)


def load_config(model_dir: str) -> ModelConfig:
    """Read `model_dir/config.json` and return the typed configuration of the architecture it
    names.  The class is chosen by the registry, never by the caller."""
    return config_from_normalised(core.call("global", None, "load_config", model_dir=model_dir))


def save_config(cfg: ModelConfig, model_dir: str) -> str:
    return core.call("global", None, "save_config", config=cfg.to_dict(), model_dir=model_dir)
