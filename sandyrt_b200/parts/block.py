"""Block arrangements.

"pre_norm": x += mixer(norm_1(x)); x += feed_forward(norm_2(x))
(src/models/gpt2_small.sandy.go:34-45 of the reference).  Norm names: "mixer", "feed_forward".
"""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import Block, LayerCallCtx, StepContext
from .linear import LazyNorm


class PreNormBlock(Block):
    norm_names = ("mixer", "feed_forward")

    def forward(self, ctx: StepContext, x: torch.Tensor, call: LayerCallCtx) -> None:
        # Parts that say `accepts_lazy_norm` get the norm unevaluated and may run it inside
        # their first product; the others get the normed tensor.
        h = LazyNorm(ctx, self.norms["mixer"], x, ctx.compute_dtype)
        self.mixer.forward(ctx, h if getattr(self.mixer, "accepts_lazy_norm", False) else h.tensor(), x, call)
        h = LazyNorm(ctx, self.norms["feed_forward"], x, ctx.compute_dtype)
        self.feed_forward.forward(ctx, h if getattr(self.feed_forward, "accepts_lazy_norm", False) else h.tensor(), x)


register_part("block", "pre_norm", PreNormBlock)
