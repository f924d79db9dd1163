"""Linear: one weight matrix with its bias, and the choice of the kernel that multiplies by it.

The weight file may store a matrix as [in, out] (GPT-2's Conv1D layout; the reference
transposes these offline, scripts/run_gpt2.py:177-189) or as [out, in].  Both are read as
they are: the 32-bit kernel takes either layout, and for the tensor-core kernels the matrix
is brought into [out, in] once, when it is bound, which is the K-major operand layout those
kernels read.

Kernel choice per call, by dtype and row count: float32 -> the FFMA kernel; bfloat16 with up
to 64 rows (a decode step) -> the weight-streaming kernel, which can also run the norm before
the product and write key/value columns into the cache; bfloat16 with more rows -> tcgen05.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorRequest


class LazyNorm:
    """A normed view of the residual stream that has not been computed yet.  A consumer either
    asks for the tensor (`tensor()`, computed once and shared) or, if its kernel can run the
    norm itself, reads `x` and `norm` and never materialises it."""

    def __init__(self, ctx, norm, x: torch.Tensor, out_dtype: torch.dtype):
        self.ctx, self.norm, self.x, self.out_dtype = ctx, norm, x, out_dtype
        self._tensor: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.x.shape

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            h = self.ctx.workspace.get("normed", self.x.shape[0], self.x.shape[1], self.out_dtype)
            self.norm.forward(self.ctx, self.x, h)
            self._tensor = h
        return self._tensor


@dataclasses.dataclass
class KVTarget:
    """Where the key/value columns of a fused q/k/v product belong: the layer's cache views and
    the step's index arrays.  `written` is set by the product if its kernel did the write."""
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    block_table: torch.Tensor
    token_seq: torch.Tensor
    positions: torch.Tensor
    q_cols: int
    kv_cols: int
    head_dim: int
    written: bool = False


class Linear:
    def __init__(self, in_features: int, out_features: int, *, bias: bool, layout: str, name: str):
        if layout not in ("in_out", "out_in"):
            raise ValueError(f"linear layout must be 'in_out' or 'out_in', got {layout!r}")
        self.in_features, self.out_features = in_features, out_features
        self.has_bias, self.layout, self.name = bias, layout, name
        self.weight: Optional[torch.Tensor] = None      # as bound; see w_out_in
        self.bias: Optional[torch.Tensor] = None
        self.w_out_in = layout == "out_in"
        self.use_tensor_cores = False

    def requests(self) -> Dict[str, TensorRequest]:
        shape = (self.in_features, self.out_features) if self.layout == "in_out" \
            else (self.out_features, self.in_features)
        req = {self.name + ".weight": TensorRequest(shape, init="weight")}
        if self.has_bias:
            req[self.name + ".bias"] = TensorRequest((self.out_features,), init="bias")
        return req

    def bind(self, tensors: Dict[str, torch.Tensor], device, dtype: torch.dtype,
             shared_weight: Optional[torch.Tensor] = None) -> None:
        """`shared_weight`: a device tensor already bound elsewhere (a tied table)."""
        if shared_weight is not None:
            w = shared_weight
        else:
            w = tensors[self.name + ".weight"].to(device=device, dtype=dtype)
        self.use_tensor_cores = (dtype == torch.bfloat16 and ops.tensor_core_gemm_supported(
            self.in_features, self.out_features))
        if self.use_tensor_cores and not self.w_out_in:
            w = w.t().contiguous()       # one-time repack to [out, in]
            self.w_out_in = True
        self.weight = w.contiguous()
        if self.has_bias:
            self.bias = tensors[self.name + ".bias"].to(device=device, dtype=dtype).contiguous()

    def weight_bytes(self) -> int:
        n = self.weight.numel() * self.weight.element_size()
        if self.bias is not None:
            n += self.bias.numel() * self.bias.element_size()
        return n

    def __call__(self, a, out: torch.Tensor, *, act: Optional[str] = None,
                 residual: Optional[torch.Tensor] = None, kv: Optional[KVTarget] = None) -> None:
        """out = act(a @ W + b) + residual.  `out` may be `residual` itself.  `a` is a tensor or a
        LazyNorm.  If `kv` is given and the kernel used can write keys/values into the cache, it
        does and sets `kv.written`; otherwise the caller appends them itself."""
        rows = a.shape[0]
        if self.use_tensor_cores and rows <= ops.SKINNY_MAX_ROWS:
            norm = None
            if isinstance(a, LazyNorm):
                if ops.skinny_norm_fusable(a, self.in_features):
                    norm = a
                    a = None
                else:
                    a = a.tensor()
            if norm is None and kv is None and \
                    ops.small_gemm_prefers_tc(rows, self.out_features, self.in_features):
                ops.gemm_tc(a, self.weight, self.bias, out, act=act, residual=residual, tile_n=64)
                return
            ops.gemm_skinny(a, self.weight, self.bias, out, act=act, residual=residual, norm=norm, kv=kv)
            if kv is not None:
                kv.written = True
            return
        if isinstance(a, LazyNorm):
            a = a.tensor()
        if self.use_tensor_cores:
            fused_kv = kv is not None and kv.head_dim % 16 == 0 and kv.q_cols % 8 == 0
            ops.gemm_tc(a, self.weight, self.bias, out, act=act, residual=residual, kv=kv if fused_kv else None)
            if fused_kv:
                kv.written = True
        else:
            ops.gemm_simt(a, self.weight, self.bias, out, w_out_in=self.w_out_in, act=act, residual=residual)
