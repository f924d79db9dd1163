"""LayerNorm part (kind "layernorm"): statistics in 32-bit, eps and width as parameters.

Formula: src/core/TensorCalc.cpp:2048-2072 of the reference (biased variance, two passes,
1/sqrt(var + eps), then gamma and beta).  Parameters: width, eps, bias (whether beta exists).
Tensors: "weight" [width], "bias" [width].
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import Norm, StepContext


class LayerNorm(Norm):
    fusable_kind = "layernorm"     # kernels that can run a norm inside themselves recognise it by this

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self._param("width"))
        self.eps = float(self._param("eps"))
        self.has_bias = bool(self._param("bias", default=True))
        self.gamma: Optional[torch.Tensor] = None
        self.beta: Optional[torch.Tensor] = None

    def requests(self) -> Dict[str, TensorRequest]:
        req = {"weight": TensorRequest((self.width,), init="gamma")}
        if self.has_bias:
            req["bias"] = TensorRequest((self.width,), init="beta")
        return req

    def bind(self, tensors, device, dtype) -> None:
        self.gamma = tensors["weight"].to(device=device, dtype=dtype).contiguous()
        self.beta = tensors["bias"].to(device=device, dtype=dtype).contiguous() if self.has_bias else None

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.gamma, self.beta) if t is not None)

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        ops.layernorm(x, self.gamma, self.beta, self.eps, out, rows=rows)


register_part("norm", "layernorm", LayerNorm)
