"""Linear: one weight matrix with its bias, and the choice of the kernel that multiplies by it.

The weight file may store a matrix as [in, out] (GPT-2's Conv1D layout; the reference
transposes these offline, scripts/run_gpt2.py:177-189) or as [out, in].  Both are read as
they are: the 32-bit kernel takes either layout, and for the tensor-core kernel the matrix
is brought into [out, in] once, when it is bound, which is the K-major operand layout that
kernel reads.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorRequest


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

    def __call__(self, a: torch.Tensor, out: torch.Tensor, *, act: Optional[str] = None,
                 residual: Optional[torch.Tensor] = None) -> None:
        """out = act(a @ W + b) + residual.  `out` may be `residual` itself."""
        if self.use_tensor_cores:
            if a.shape[0] <= ops.SKINNY_MAX_ROWS:
                ops.gemm_skinny(a, self.weight, self.bias, out, act=act, residual=residual)
            else:
                ops.gemm_tc(a, self.weight, self.bias, out, act=act, residual=residual)
        else:
            ops.gemm_simt(a, self.weight, self.bias, out, w_out_in=self.w_out_in, act=act, residual=residual)
