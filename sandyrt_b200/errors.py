"""The engine's exception classes.

The host library reports every failure with the name of its kind; the binding raises the class of
that name.  `ValueError` and `RuntimeError` kinds map to Python's own.
"""
from __future__ import annotations

import json
from typing import List, Tuple


class ConfigError(ValueError):
    """A config.json that is missing, malformed or names impossible sizes."""


class WeightFileError(Exception):
    """The weight file is missing, truncated or not a well-formed safetensors file."""


class WeightBindingError(Exception):
    """The weight file does not hold exactly the tensors the model needs.  The message lists
    everything; the parts are in `missing`, `unexpected`, `wrong_shape` [(name, got, want)] and
    `wrong_kind` [(name, dtype)]."""

    def __init__(self, message: str, details: str = ""):
        super().__init__(message)
        d = json.loads(details) if details else {}
        self.path: str = d.get("path", "")
        self.missing: List[str] = list(d.get("missing", []))
        self.unexpected: List[str] = list(d.get("unexpected", []))
        self.wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]] = [
            (n, tuple(got), tuple(want)) for n, got, want in d.get("wrong_shape", [])]
        self.wrong_kind: List[Tuple[str, str]] = [(n, k) for n, k in d.get("wrong_kind", [])]


class CacheError(Exception):
    """A misuse of the cache: unknown request, page freed twice, shrinking a request..."""


class OutOfPages(Exception):
    """A group's pool cannot supply the pages a reservation needs.  Nothing was taken."""


class NoFreeSlot(Exception):
    """Every state slot is held by a live request."""


class RequestRefused(ValueError):
    """The request can never be served (empty prompt, too long for the model or the pool)."""


class StepError(Exception):
    """A step that cannot run as given, or bad input reported by a kernel."""


class KernelError(RuntimeError):
    pass


class UnsupportedShape(KernelError):
    pass


class KernelBuildError(RuntimeError):
    pass


class ForeignError(RuntimeError):
    """A part or architecture defined outside the host library failed."""


KINDS = {c.__name__: c for c in (ConfigError, WeightFileError, WeightBindingError, CacheError, OutOfPages, NoFreeSlot,
                                 RequestRefused, StepError, KernelError, UnsupportedShape, KernelBuildError, ForeignError)}
KINDS.update({"ValueError": ValueError, "RuntimeError": RuntimeError, "MemoryError": MemoryError})
