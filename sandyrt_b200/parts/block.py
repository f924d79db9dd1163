"""Block arrangements.

"pre_norm": x += mixer(norm_1(x)); x += feed_forward(norm_2(x))
(src/models/gpt2_small.sandy.go:34-45 of the reference).  Norm names: "mixer", "feed_forward".
"""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import Block, LayerCallCtx, StepContext


class PreNormBlock(Block):
    norm_names = ("mixer", "feed_forward")

    def forward(self, ctx: StepContext, x: torch.Tensor, call: LayerCallCtx) -> None:
        h = ctx.workspace.get("normed", x.shape[0], self.width, ctx.compute_dtype)
        self.norms["mixer"].forward(ctx, x, h)
        self.mixer.forward(ctx, h, x, call)
        self.norms["feed_forward"].forward(ctx, x, h)
        self.feed_forward.forward(ctx, h, x)


register_part("block", "pre_norm", PreNormBlock)
