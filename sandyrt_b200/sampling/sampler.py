"""Sampler: turns a step's logits into one token per sampled row, on the device.

The uniform number behind every draw comes from a counter-based generator keyed by the
request's seed and the index of the token being drawn, so a request's tokens do not depend
on which other requests share its steps.  (The reference draws on the host from one
std::mt19937_64 per sampler, src/server/Sampler.cpp:127-131, serving one request at a time.)
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams

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


class Sampler:
    def __init__(self, device):
        self.device = device
        self._cap = 0
        self._host = None
        self._dev = None
        self._tokens = None
        self._status = torch.zeros(1, dtype=torch.int32, device=device)

    def _ensure(self, n: int) -> None:
        if n <= self._cap:
            return
        self._cap = max(64, 1 << (n - 1).bit_length())
        self._host = torch.empty((4, self._cap), dtype=torch.float32, pin_memory=True)
        self._dev = torch.empty((4, self._cap), dtype=torch.float32, device=self.device)
        self._tokens = torch.empty(self._cap, dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               seeds: Sequence[int], indices: Sequence[int]) -> torch.Tensor:
        """logits: float32 [n, vocab] on the device.  Row i is drawn with params[i]; its
        uniform number is uniform_for(seeds[i], indices[i]).  Returns int32 [n] on the device."""
        n = logits.shape[0]
        self._ensure(n)
        tokens = self._tokens[:n]
        if all(p.greedy for p in params):
            ops.sample(logits, tokens, status=self._status)
            return tokens
        h = self._host.numpy()
        for i, p in enumerate(params):
            h[0, i] = 0.0 if p.greedy else p.temperature
            h[2, i] = p.top_p
            h[3, i] = uniform_for(seeds[i], indices[i])
        hk = self._host.view(torch.int32).numpy()
        for i, p in enumerate(params):
            hk[1, i] = p.top_k
        # The host buffer is reused every call: the caller reads the drawn tokens back (a
        # stream-ordered wait) before it samples again, so the previous copy is over by now.
        self._dev[:, :n].copy_(self._host[:, :n], non_blocking=True)
        d = self._dev
        ops.sample(logits, tokens, temperature=d[0, :n], top_k=d[1, :n].view(torch.int32),
                   top_p=d[2, :n], uniform=d[3, :n], status=self._status)
        return tokens

    def check_status(self) -> None:
        if int(self._status.item()):
            self._status.zero_()
            raise ValueError("sampling logits must not contain NaN")   # Sampler.cpp:64-67
