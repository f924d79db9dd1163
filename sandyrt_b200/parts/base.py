"""Interfaces of the parts a model is put together from, and the per-step context they see.

A part is built from a PartSpec (its kind, its sizes and constants, the names of its
tensors), says which tensors it needs (`requests`), receives them (`bind`) and then runs
on the tokens of a step (`forward`).  It knows its own sizes and nothing of the model it
sits in: layer indices, architecture names and config.json keys never reach it.

Families and what each must provide:

  Norm            forward(ctx, x, out_dtype, rows=None) -> y
  PositionEncoding
                  table() -> tensor added to the token embedding, or None
                  rotate(ctx, q, k) -> None (in place), for encodings applied to queries and keys
                  max_positions -> int or None
  Mixer           cache_spec() -> PagedKVSpec | StateSpec | None
                  forward(ctx, h, x, call) -> None   (x += mix(h), in place)
  FeedForward     forward(ctx, h, x) -> None         (x += ff(h), in place)
  Block           forward(ctx, x, call) -> None      (runs its norms, mixer, feed-forward)
  Embedding       forward(ctx, x, status) -> None    (x = the tokens' rows, position table added)
                  table() -> the bound token table
  Head            forward(ctx, y, logits) -> None    (float32 logits of the normed rows y)

`x` is the residual stream: float32 [tokens, width] in both compute dtypes, so the
residual sum is always formed and kept in 32-bit.  `h` is a normed copy in the compute
dtype (float32 or bfloat16).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..models.spec import PartSpec
from ..weights.loader import TensorRequest, to_device


# ---- what a mixer may ask of the cache manager ---------------------------------------
@dataclasses.dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every position (or of the last `window` positions) in pages."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None   # None: all positions stay; n: only the last n are read


@dataclasses.dataclass(frozen=True)
class StateSpec:
    """A per-request state of fixed size (a recurrent state, a convolution tail, ...).
    It lives in the request's state slot, starts as zeros when the request is admitted
    and is float32 unless `dtype` says otherwise."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclasses.dataclass
class LayerCallCtx:
    """Which cache entry the running layer call works on."""
    cache: int
    write_cache: bool


class Workspace:
    """Named scratch tensors that keep their address from step to step (so that a captured
    CUDA graph stays valid) and only ever grow."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.version = 0      # bumped whenever a buffer moves; recorded graphs check it

    def get(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, dtype)
        need = rows * cols
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < need:
            buf = torch.empty(max(need, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.version += 1
        return buf[:need].view(rows, cols)

    def reserve(self, name: str, numel: int, dtype: torch.dtype) -> None:
        self.get(name, 1, numel, dtype)


@dataclasses.dataclass
class StepContext:
    """Everything a part may read about the running step.  Device tensors are int32."""
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor          # [T] the step's tokens, requests back to back
    positions: torch.Tensor          # [T] position of each token in its request
    token_seq: torch.Tensor          # [T] which of the step's requests a token belongs to
    seq_slots: torch.Tensor          # [S] state slot of each request
    q_start: torch.Tensor            # [S+1] first token of each request in the step
    kv_before: torch.Tensor          # [S] tokens each request had before the step
    logit_rows: torch.Tensor         # [R] tokens whose logits are wanted
    block_tables: Dict[int, torch.Tensor]   # cache group -> [S, max_blocks]
    compute_dtype: torch.dtype
    workspace: Workspace
    caches: Any                      # cache.manager.DeviceCaches: kv(cache) / state(cache)
    position: Any = None             # the model's PositionEncoding
    # host copies, for parts that plan their launches on the host
    host_q_lens: List[int] = dataclasses.field(default_factory=list)
    host_kv_before: List[int] = dataclasses.field(default_factory=list)
    host_slots: List[int] = dataclasses.field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0


class Part:
    """Base of every part: tensor requests and binding."""

    # A part whose `forward` only launches kernels that read the step's device arrays may be
    # recorded in a CUDA graph and replayed.  A part that decides anything from the step's
    # host-side lists (ctx.host_*) must set this to False; the engine then runs every step of
    # a model that holds such a part without graphs.
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
        """Bytes of weights one step reads from this part (used for roofline figures); parts
        with matrices override it."""
        return 0

    # helpers ---------------------------------------------------------------------------
    def _param(self, key: str, kind=None, default=dataclasses.MISSING):
        if key not in self.params:
            if default is dataclasses.MISSING:
                raise KeyError(f"{type(self).__name__}: parameter '{key}' is required")
            return default
        return self.params[key]


class Norm(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    max_positions: Optional[int] = None
    rotates = False      # True for encodings that act on queries and keys (`rotate`)

    def table(self) -> Optional[torch.Tensor]:
        return None

    def rotate(self, ctx: StepContext, q: torch.Tensor, k: Optional[torch.Tensor]) -> None:
        return None


class Embedding(Part):
    """Token ids to the first residual stream.  `table()` is the bound token table (a head that
    is tied to it multiplies by the same tensor)."""

    def table(self) -> Optional[torch.Tensor]:
        return None

    def forward(self, ctx: "StepContext", x: torch.Tensor, status: Optional[torch.Tensor]) -> None:
        raise NotImplementedError


class Head(Part):
    """The last normed rows to float32 logits.  `tied` says that it shares the embedding's table
    (its `bind` then receives `tied_weight`)."""
    tied = False

    def bind(self, tensors, device, dtype, tied_weight: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError

    def forward(self, ctx: "StepContext", y: torch.Tensor, logits: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor, call: LayerCallCtx) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor) -> None:
        raise NotImplementedError


class Block:
    """An arrangement of norms, a mixer and a feed-forward (built from a LayerSpec)."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm], width: int):
        self.mixer, self.feed_forward, self.norms, self.width = mixer, feed_forward, norms, width

    def forward(self, ctx: StepContext, x: torch.Tensor, call: LayerCallCtx) -> None:
        raise NotImplementedError
