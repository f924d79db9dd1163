"""Base classes for parts defined in Python (the engine's own parts live in the host library)."""
from .base import (FeedForward, LayerCallCtx, Mixer, Norm, PagedKVSpec, Part, PositionEncoding,  # noqa: F401
                   StateSpec, StepContext)
