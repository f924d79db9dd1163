"""A test bench for one of the host library's parts outside a model (core/harness.cpp).

It builds the part from its description, binds seeded random tensors (whose values it hands back,
for the reference computation), keeps a small cache of its own and runs the part over hand-made
steps on torch tensors.  Tests compare each part alone with the plain implementation's function
for it.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import core
from ..models.spec import PartSpec

_DTYPE_NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


class PartHarness:
    def __init__(self, family: str, spec: PartSpec, dtype: torch.dtype = torch.float32, *,
                 position: Optional[PartSpec] = None, page_size: int = 8, max_tokens: int = 512, max_requests: int = 8,
                 seed: int = 0):
        self._h = core.Handle("harness", core.call(
            "global", None, "new_harness", family=family, part=spec.to_json(),
            position=None if position is None else position.to_json(), dtype=_DTYPE_NAMES[dtype], page_size=page_size,
            max_tokens=max_tokens, max_requests=max_requests, seed=seed)["handle"])

    def _values(self, table) -> Dict[str, np.ndarray]:
        out = {}
        for name, e in table.items():
            n = int(np.prod(e["shape"])) if e["shape"] else 1
            raw = (ctypes.c_float * n).from_address(e["address"])
            out[name] = np.frombuffer(raw, dtype=np.float32).reshape(e["shape"]).copy()
        return out

    def tensors(self) -> Dict[str, np.ndarray]:
        """The float32 values the part was bound with, by its own tensor names."""
        return self._values(self._h.call("tensors")["part"])

    def position_tensors(self) -> Dict[str, np.ndarray]:
        return self._values(self._h.call("tensors")["position"])

    def info(self) -> dict:
        return self._h.call("info")

    def set_step(self, seqs: Sequence[Tuple[int, int]], ids: Optional[Sequence[int]] = None) -> None:
        """The next step: for each request (tokens before, new tokens).  A request seen before moves
        on: its earlier tokens are committed and the new ones reserved."""
        self._h.call("set_step", seqs=[[int(b), int(n)] for b, n in seqs], ids=None if ids is None else [int(t) for t in ids])

    def run_norm(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[Sequence[int]] = None) -> None:
        torch.cuda.synchronize()
        self._h.call("run_norm", x=x.data_ptr(), x_rows=x.shape[0], out=out.data_ptr(), n_rows=out.shape[0],
                     rows=None if rows is None else [int(r) for r in rows])

    def run_feed_forward(self, h: torch.Tensor, x: torch.Tensor) -> None:
        torch.cuda.synchronize()
        self._h.call("run_feed_forward", h=h.data_ptr(), x=x.data_ptr())

    def run_mixer(self, h: torch.Tensor, x: torch.Tensor, write_cache: bool = True) -> None:
        torch.cuda.synchronize()
        self._h.call("run_mixer", h=h.data_ptr(), x=x.data_ptr(), write_cache=write_cache)

    def run_embedding(self, x: torch.Tensor) -> None:
        torch.cuda.synchronize()
        self._h.call("run_embedding", x=x.data_ptr())
