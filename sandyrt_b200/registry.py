"""Registries: architecture name -> model description, and part kind -> part class.

The reference picks a model by an if/else chain over an `architecture` string
(src/server/Model.cpp:100-160, unknown -> "unknown model architecture: X").  Here both
the architectures and the parts they are built from are entries of open tables, so a
new mixer, feed-forward, norm, position encoding or whole architecture is added by
registering it; no file of the framework changes.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, Type

from .config.base import ConfigError, ModelConfig


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    # describe(config) -> ModelSpec (see models/spec.py): the parts of every layer, the
    # order in which layers run, and the names of the tensors in the weight file.
    describe: Callable[[ModelConfig], "object"]


_ARCHITECTURES: Dict[str, Architecture] = {}
_PART_KINDS = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_PARTS: Dict[str, Dict[str, type]] = {k: {} for k in _PART_KINDS}


def register_architecture(name: str, config_cls: Type[ModelConfig], describe) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_cls, describe)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown model architecture: {name!r}; registered: {sorted(_ARCHITECTURES)}") from None


def architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def register_part(family: str, kind: str, cls: type) -> None:
    """Register class `cls` as the implementation of part `kind` in `family`
    ("mixer", "feed_forward", "norm", "position", "block", "embedding" or "head")."""
    if family not in _PARTS:
        raise KeyError(f"unknown part family {family!r}; one of {_PART_KINDS}")
    _PARTS[family][kind] = cls


def get_part(family: str, kind: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[family][kind]
    except KeyError:
        raise ConfigError(
            f"unknown {family} kind {kind!r}; registered: {sorted(_PARTS.get(family, {}))}") from None


_BUILTIN_DONE = False


def _ensure_builtin() -> None:
    """Import the modules that register the parts and architectures shipped here."""
    global _BUILTIN_DONE
    if _BUILTIN_DONE:
        return
    _BUILTIN_DONE = True
    from . import parts  # noqa: F401  (registers built-in part kinds)
    from . import models  # noqa: F401  (registers built-in architectures)
