"""Token embedding and output head.

TokenEmbedding: x[t] = table[id[t]] (+ position table[pos[t]] when the position encoding
has one), one fused pass (src/models/gpt2_small.sandy.go:48-50 of the reference).

OutputHead: logits = y @ W^T in float32.  With `tied` the token table itself is the
weight: the reference ties by naming `wte.weight` twice (:57, a transposed-operand matmul,
src/ir/MidIRPass.cpp:30-69), and no second copy exists here either.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..models.spec import PartSpec
from ..weights.loader import TensorRequest
from ..registry import register_part
from .base import Embedding, Head, StepContext
from .linear import Linear


class TokenEmbedding(Embedding):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.vocab_size = int(self._param("vocab_size"))
        self.width = int(self._param("width"))
        self.weight: Optional[torch.Tensor] = None

    def requests(self) -> Dict[str, TensorRequest]:
        return {"weight": TensorRequest((self.vocab_size, self.width), init="weight")}

    def bind(self, tensors, device, dtype) -> None:
        self.weight = tensors["weight"].to(device=device, dtype=dtype).contiguous()

    def table(self) -> Optional[torch.Tensor]:
        return self.weight

    def weight_bytes(self) -> int:
        return 0        # a step reads a few rows of the table, not the table

    def forward(self, ctx: StepContext, x: torch.Tensor, status: Optional[torch.Tensor]) -> None:
        table = ctx.position.table() if ctx.position is not None else None
        ops.embed_positions(ctx.token_ids, ctx.positions, self.weight, table, x, status=status)


class OutputHead(Head):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.vocab_size = int(self._param("vocab_size"))
        self.width = int(self._param("width"))
        self.tied = bool(self._param("tied"))
        self.linear = Linear(self.width, self.vocab_size, bias=False, layout="out_in", name="head")

    def requests(self) -> Dict[str, TensorRequest]:
        if self.tied:
            return {}
        return {"weight": TensorRequest((self.vocab_size, self.width), init="weight")}

    def bind(self, tensors, device, dtype, tied_weight: Optional[torch.Tensor] = None) -> None:
        if self.tied:
            if tied_weight is None:
                raise ValueError("tied output head needs the token table")
            self.linear.bind({}, device, dtype, shared_weight=tied_weight)
        else:
            self.linear.bind({"head.weight": tensors["weight"]}, device, dtype)

    def forward(self, ctx: StepContext, y: torch.Tensor, logits: torch.Tensor) -> None:
        self.linear(y, logits)

    def weight_bytes(self) -> int:
        return self.linear.weight_bytes()


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "output_head", OutputHead)
