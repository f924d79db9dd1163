"""Causal self-attention over the paged cache (kind "causal_attention").

  qkv = h @ W_qkv + b_qkv;  q, k, v = column ranges [0, H*D), [H*D, (H+Hkv)*D), the rest
  (k, v) of the step's tokens are appended to the request's pages
  o = attention(q, all cached k, v up to each token's own position)
  x += o @ W_out + b_out
Formulas: src/models/gpt2_small.sandy.go:1-23 and src/core/TensorCalc.cpp:1241-1311 of the
reference (which splits the fused matrix offline into q/k/v, scripts/run_gpt2.py:170-175;
here the fused matrix is used as stored and the split is three column ranges).

Parameters: width, n_heads, n_kv_heads, head_dim, scale (the factor on q.k, already
including any per-layer factor the architecture wants), window (None = all positions),
bias, weight_layout.  Tensors: "qkv.weight", "qkv.bias", "out.weight", "out.bias".
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import LayerCallCtx, Mixer, PagedKVSpec, StepContext
from .linear import KVTarget, Linear


class CausalSelfAttention(Mixer):
    accepts_lazy_norm = True     # `h` may arrive as a LazyNorm; the q/k/v projection runs it

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(self._param("width"))
        self.n_heads = int(self._param("n_heads"))
        self.n_kv_heads = int(self._param("n_kv_heads", default=self.n_heads))
        self.head_dim = int(self._param("head_dim"))
        self.scale = float(self._param("scale"))
        window = self._param("window", default=None)
        self.window: Optional[int] = int(window) if window else None
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"causal_attention: {self.n_heads} heads do not divide into "
                             f"{self.n_kv_heads} key/value heads")
        if self.head_dim % 16 != 0 or not (0 < self.head_dim <= 256):
            raise ValueError(f"causal_attention: head size {self.head_dim} must be a multiple of 16, at most 256")
        bias = bool(self._param("bias", default=True))
        layout = str(self._param("weight_layout", default="out_in"))
        self.q_cols = self.n_heads * self.head_dim
        self.kv_cols = self.n_kv_heads * self.head_dim
        self.qkv = Linear(self.width, self.q_cols + 2 * self.kv_cols, bias=bias, layout=layout, name="qkv")
        self.out = Linear(self.q_cols, self.width, bias=bias, layout=layout, name="out")

    def requests(self) -> Dict[str, TensorRequest]:
        return {**self.qkv.requests(), **self.out.requests()}

    def bind(self, tensors, device, dtype) -> None:
        self.qkv.bind(tensors, device, dtype)
        self.out.bind(tensors, device, dtype)

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor, call: LayerCallCtx) -> None:
        T = h.shape[0]
        ws = ctx.workspace
        qkv = ws.get("qkv", T, self.q_cols + 2 * self.kv_cols, ctx.compute_dtype)
        k_cache, v_cache, group = ctx.caches.kv(call.cache)
        table = ctx.block_tables[group]
        rotates = ctx.position is not None and getattr(ctx.position, "rotates", False)
        # keys/values may go straight from the projection's write-back into the pages, unless
        # a position encoding still has to turn them first
        target = None
        if call.write_cache and not rotates:
            target = KVTarget(k_cache, v_cache, table, ctx.token_seq, ctx.positions, self.q_cols, self.kv_cols,
                              self.head_dim)
        self.qkv(h, qkv, kv=target)
        q = qkv[:, :self.q_cols]
        k = qkv[:, self.q_cols:self.q_cols + self.kv_cols]
        v = qkv[:, self.q_cols + self.kv_cols:]
        if rotates:
            ctx.position.rotate(ctx, q, k if call.write_cache else None)
        if call.write_cache and not (target is not None and target.written):
            ops.kv_append(k, v, k_cache, v_cache, table, ctx.token_seq, ctx.positions)
        o = ws.get("attn_out", T, self.q_cols, ctx.compute_dtype)
        ops.attention(ctx, q, k_cache, v_cache, table, o, n_heads=self.n_heads, scale=self.scale,
                      window=self.window or 0)
        self.out(o, x, residual=x)

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.out.weight_bytes()


register_part("mixer", "causal_attention", CausalSelfAttention)
