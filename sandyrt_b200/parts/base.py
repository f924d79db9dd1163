"""Parts defined in Python: the base classes a caller subclasses, and the step as such a part sees it.

The engine's own parts (LayerNorm, causal attention over the paged cache, the dense feed-forward,
learned positions, the pre-norm block, token embedding and output head) are C++ classes of the host
library (core/parts.cpp).  A caller can add a mixer, feed-forward, norm or position encoding of its
own WITHOUT touching the library: subclass one of the classes below, register it
(registry.register_part) and name its kind in a model description.  The library then builds it,
asks it for its tensors, binds them and calls its `forward` through callbacks, on the engine's
stream, with device memory wrapped as torch tensors.

What each family must provide:

  Mixer             cache_spec() -> PagedKVSpec | StateSpec | None
                    forward(ctx, h, x, call) -> None      (x += mix(h), in place)
  FeedForward       forward(ctx, h, x) -> None            (x += ff(h), in place)
  Norm              forward(ctx, x, out, rows=None) -> None
  PositionEncoding  rotates / rotate(ctx, q, k) -> None   (in place on queries and keys)
                    max_positions -> int or None

`x` is the residual stream: float32 [tokens, width] in both compute dtypes.  `h` is a normed copy
in the compute dtype.  Set `graph_safe = False` on a part that plans its work from the step's
host-side lists (ctx.host_*): the engine then runs every step of a model holding it without graphs.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import core
from ..models.spec import PartSpec
from ..weights.loader import TensorRequest


# ---- what a mixer may ask of the cache manager ---------------------------------------
@dataclasses.dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every position (or of the last `window` positions) in pages."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None   # None: all positions stay; n: only the last n are read

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "paged", "n_kv_heads": self.n_kv_heads, "head_dim": self.head_dim, "window": self.window or 0}


@dataclasses.dataclass(frozen=True)
class StateSpec:
    """A per-request state of fixed size (a recurrent state, a convolution tail, ...).  It lives in
    the request's state slot, starts as zeros when the request is admitted and is float32 unless
    `dtype` says otherwise."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "state", "shape": list(self.shape),
                "dtype": {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.int32: "int32"}[self.dtype]}


def cache_spec_json(spec) -> Optional[Dict[str, Any]]:
    return None if spec is None else spec.to_json()


@dataclasses.dataclass
class LayerCallCtx:
    """Which cache entry the running layer call works on."""
    cache: int
    write_cache: bool


# ---- device memory as torch tensors -------------------------------------------------------
_TORCH_DTYPES = {0: torch.float32, 1: torch.bfloat16, 2: torch.int32}
_TYPESTR = {0: "<f4", 1: "<i2", 2: "<i4"}
_ELEM = {0: 4, 1: 2, 2: 4}


class _DeviceArray:
    def __init__(self, ptr: int, shape: Tuple[int, ...], code: int, strides_bytes: Optional[Tuple[int, ...]] = None):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": tuple(shape), "typestr": _TYPESTR[code],
                                         "version": 2, "strides": strides_bytes}


def wrap_device(ptr: int, shape: Tuple[int, ...], code: int, strides: Optional[Tuple[int, ...]] = None) -> torch.Tensor:
    """A torch tensor over device memory the library owns (no copy).  `strides` in elements."""
    if any(d == 0 for d in shape) or not ptr:
        return torch.empty(shape, dtype=_TORCH_DTYPES[code], device="cuda")
    sb = None if strides is None else tuple(s * _ELEM[code] for s in strides)
    t = torch.as_tensor(_DeviceArray(ptr, shape, code, sb), device="cuda")
    return t.view(torch.bfloat16) if code == 1 else t


def wrap_view(view: "core.TensorView") -> torch.Tensor:
    return wrap_device(view.data, (view.rows, view.cols), view.dtype, (view.ld, 1))


class StepCaches:
    """The step's cache entries as a part defined in Python sees them."""

    def __init__(self, step_ptr):
        self._step = step_ptr

    def state(self, cache: int) -> torch.Tensor:
        """The fixed-size state of a cache entry, [max_requests, elements]; row `slot` is a request's."""
        v = core.TensorView()
        if core.lib().sandy_step_state(self._step, ctypes.c_int(cache), ctypes.byref(v)) != 0:
            core.raise_last_error()
        return wrap_device(v.data, (v.rows, v.cols), v.dtype)

    def kv(self, cache: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
        """(K view, V view, group) of a cache entry; views are [num_pages, Hkv, page_size, D]."""
        k, v = core.TensorView(), core.TensorView()
        group, hkv, ps, d = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        if core.lib().sandy_step_kv(self._step, ctypes.c_int(cache), ctypes.byref(k), ctypes.byref(v), ctypes.byref(group),
                                    ctypes.byref(hkv), ctypes.byref(ps), ctypes.byref(d)) != 0:
            core.raise_last_error()
        shape = (k.rows, hkv.value, ps.value, d.value)
        strides = (k.ld, ps.value * d.value, d.value, 1)
        return wrap_device(k.data, shape, k.dtype, strides), wrap_device(v.data, shape, v.dtype, strides), group.value


class StepContext:
    """Everything a part may read about the running step.  Device tensors are int32."""

    def __init__(self, step_ptr):
        s = step_ptr.contents
        T, S, R = s.n_tokens, s.n_seqs, s.n_rows
        self.n_tokens, self.n_seqs = T, S
        self.token_ids = wrap_device(s.token_ids, (T,), 2)        # [T] the step's tokens, requests back to back
        self.positions = wrap_device(s.positions, (T,), 2)        # [T] position of each token in its request
        self.token_seq = wrap_device(s.token_seq, (T,), 2)        # [T] which of the step's requests a token belongs to
        self.seq_slots = wrap_device(s.seq_slots, (S,), 2)        # [S] state slot of each request
        self.q_start = wrap_device(s.q_start, (S + 1,), 2)        # [S+1] first token of each request in the step
        self.kv_before = wrap_device(s.kv_before, (S,), 2)        # [S] tokens each request had before the step
        self.logit_rows = wrap_device(s.logit_rows, (R,), 2)      # [R] tokens whose logits are wanted
        self.block_tables = {g: wrap_device(s.block_tables[g], (S, s.max_blocks), 2) for g in range(s.n_groups)}
        self.compute_dtype = _TORCH_DTYPES[s.compute_dtype]
        self.caches = StepCaches(step_ptr)
        # host copies, for parts that plan their launches on the host
        self.host_q_lens: List[int] = [s.host_q_lens[i] for i in range(S)]
        self.host_kv_before: List[int] = [s.host_kv_before[i] for i in range(S)]
        self.host_slots: List[int] = [s.host_slots[i] for i in range(S)]
        self.max_q_len, self.max_kv_len = s.max_q_len, s.max_kv_len
        self.stream = s.stream


class Part:
    """Base of every part defined in Python: tensor requests and binding."""

    graph_safe = True

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.params: Dict[str, Any] = dict(spec.params)

    def requests(self) -> Dict[str, TensorRequest]:
        """Local tensor name -> what is expected of it."""
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        """Receive the tensors named by `requests` (host tensors) and place them on the device."""

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads from this part (for roofline figures)."""
        return 0


class Norm(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    max_positions: Optional[int] = None
    rotates = False      # True for encodings that act on queries and keys (`rotate`)

    def rotate(self, ctx: StepContext, q: torch.Tensor, k: Optional[torch.Tensor]) -> None:
        return None


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor, call: LayerCallCtx) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor) -> None:
        raise NotImplementedError
