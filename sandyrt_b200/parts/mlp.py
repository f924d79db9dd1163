"""Dense feed-forward (kind "dense_mlp"): up-projection, activation, down-projection.

  u = h @ W_up + b_up;  g = act(u);  x += g @ W_down + b_down
(src/models/gpt2_small.sandy.go:25-32,40-42 of the reference).  The activation runs in the
up-projection's write-back and the residual sum in the down-projection's, both in 32-bit.
Parameters: width, inner, activation ("gelu_new" | "gelu"), bias, weight_layout.
Tensors: "up.weight", "up.bias", "down.weight", "down.bias".
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc.ops import ACT_CODES
from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import FeedForward, StepContext
from .linear import Linear


class DenseMLP(FeedForward):
    accepts_lazy_norm = True     # `h` may arrive as a LazyNorm; the up-projection runs it

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self._param("width"))
        self.inner = int(self._param("inner"))
        self.activation = str(self._param("activation"))
        if self.activation not in ACT_CODES or self.activation in (None, "none"):
            raise ValueError(f"dense_mlp: unknown activation {self.activation!r}")
        bias = bool(self._param("bias", default=True))
        layout = str(self._param("weight_layout", default="out_in"))
        self.up = Linear(self.width, self.inner, bias=bias, layout=layout, name="up")
        self.down = Linear(self.inner, self.width, bias=bias, layout=layout, name="down")

    def requests(self) -> Dict[str, TensorRequest]:
        return {**self.up.requests(), **self.down.requests()}

    def bind(self, tensors, device, dtype) -> None:
        self.up.bind(tensors, device, dtype)
        self.down.bind(tensors, device, dtype)

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor) -> None:
        g = ctx.workspace.get("ff_inner", h.shape[0], self.inner, ctx.compute_dtype)
        self.up(h, g, act=self.activation)
        self.down(g, x, residual=x)

    def weight_bytes(self) -> int:
        return self.up.weight_bytes() + self.down.weight_bytes()


register_part("feed_forward", "dense_mlp", DenseMLP)
