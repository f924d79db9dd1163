"""Sampling options of a request, with the reference's names and meanings.

src/server/Sampler.h:13-22 of the reference: SamplingConfig{topK = 1, topP = 1.0,
temperature = 0.0}, per-request overrides of temperature and top_p; checked by
resolveSamplingConfig (src/server/Sampler.cpp:111-125): top_k > 0, 0 < top_p <= 1,
temperature >= 0 and finite.  temperature 0 is greedy.

One difference: the reference's default top_k = 1 makes every draw greedy until a model's
model_config.json raises it (src/server/Model.cpp:63-96).  Here top_k = 0 means "no top-k
cut" and is the default, so `temperature` alone switches sampling on.

The checks are the host library's (core/sampling.h).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

from .. import core


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0             # 0: whole vocabulary
    top_p: float = 1.0
    seed: Optional[int] = None  # None: a fresh seed per request

    def validate(self) -> "SamplingParams":
        core.call("global", None, "validate_sampling", temperature=float(self.temperature), top_k=int(self.top_k),
                  top_p=float(self.top_p))
        return self

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1
