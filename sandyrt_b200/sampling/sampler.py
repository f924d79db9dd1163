"""The uniform numbers behind sampled tokens.

Drawing itself runs on the device (csrc/sampling.cu, launched by the step function).  The uniform
number behind every draw comes from a counter-based generator keyed by the request's seed and the
index of the token being drawn (core/sampling.h), so a request's tokens do not depend on which other
requests share its steps.  (The reference draws on the host from one std::mt19937_64 per sampler,
src/server/Sampler.cpp:127-131, serving one request at a time.)
"""
from __future__ import annotations

import os

from .. import core

_MASK = (1 << 63) - 1


def uniform_for(seed: int, index: int) -> float:
    """The uniform number in [0, 1) for token `index` of a request with `seed` (24 bits, so it is
    exact in float32)."""
    return float(core.call("global", None, "uniform_for", seed=int(seed) & _MASK, index=int(index)))


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little") & _MASK
