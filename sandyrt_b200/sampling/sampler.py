"""The uniform numbers behind sampled tokens.

Drawing itself runs on the device (csrc/sampling.cu, launched by the step function).  The
uniform number behind every draw comes from a counter-based generator keyed by the
request's seed and the index of the token being drawn, so a request's tokens do not depend
on which other requests share its steps.  (The reference draws on the host from one
std::mt19937_64 per sampler, src/server/Sampler.cpp:127-131, serving one request at a time.)
"""
from __future__ import annotations

import os

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_for(seed: int, index: int) -> float:
    """The uniform number in [0, 1) for token `index` of a request with `seed` (24 bits, so it
    is exact in float32)."""
    h = _splitmix64((_splitmix64(seed & _MASK) + index) & _MASK)
    return (h >> 40) / float(1 << 24)


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")
