"""Position encodings.

"learned_absolute": a table [max_positions, width] added to the token embedding
(src/models/gpt2_small.sandy.go:49-50 of the reference: a second embedding lookup with
position ids, then an add).  Positions are supplied by the step, not derived.  The table's
length is a hard limit on a request's length.

"none": no encoding at the embedding and no limit.  An encoding that acts on queries and
keys instead (a rotation) overrides `rotate` and leaves `table` as None.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import PositionEncoding


class LearnedAbsolute(PositionEncoding):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self._param("width"))
        self.max_positions = int(self._param("max_positions"))
        self._table: Optional[torch.Tensor] = None

    def requests(self) -> Dict[str, TensorRequest]:
        return {"weight": TensorRequest((self.max_positions, self.width), init="weight")}

    def bind(self, tensors, device, dtype) -> None:
        self._table = tensors["weight"].to(device=device, dtype=dtype).contiguous()

    def table(self) -> Optional[torch.Tensor]:
        return self._table


class NoPosition(PositionEncoding):
    max_positions = None


register_part("position", "learned_absolute", LearnedAbsolute)
register_part("position", "none", NoPosition)
