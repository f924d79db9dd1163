"""The step function: one batch of (request, its next tokens) through the model.

`Engine.step(entries)` takes, for each request of the step, the tokens that follow what the request
already has in the cache (a portion of a prompt of any length, or one decoded token) and the places
among them whose logits are wanted.  It runs exactly those tokens as one batch, reading everything
earlier from the cache, appends their keys and values to the cache, and returns float32 logits
[wanted, vocab] in the order of the entries and of their wanted places.  With `sampling` it also
draws one token per wanted row on the device.

The step function itself (packing the step's arrays into one pinned buffer, one copy to the device,
CUDA graphs per step shape, bursts of decode steps that feed their tokens back on the device) is
the host library's (core/engine.cpp); this class is its Python face.  The reference's counterpart,
Engine::runValues on one of two compiled graphs (src/engine/Engine.h:100-104,
src/server/Model.cpp:216-255, inputs built in src/server/Session.cpp:167-206), serves one request
per call, returns logits for every row and samples on the host.

The engine runs on a stream of its own.  `step` returns once the logits are complete; bursts are
queued and read with `burst_tokens`.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import core
from ..cache.pages import BlockAllocator, RequestIds
from ..errors import OutOfPages, StepError  # noqa: F401  (re-exported)
from ..models.model import Model
from ..parts.base import wrap_device

MAX_BURST = 32      # most decode steps one decode_burst may run


@dataclasses.dataclass
class StepEntry:
    """One request's share of a step."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()        # indices into `tokens` whose logits are returned


@dataclasses.dataclass
class SampleRow:
    """How the token of one wanted row is drawn (see sampling.params.SamplingParams)."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    uniform: float = 0.0


@dataclasses.dataclass
class BurstHandle:
    """A burst of decode steps queued on the device (Engine.decode_burst_async)."""
    n: int                       # steps
    S: int                       # requests
    burst: int                   # the library's handle


class _DeviceCachesView:
    def __init__(self, engine: "Engine"):
        self._engine = engine

    def poison(self) -> None:
        """Fill every page with NaN (tests: a read of a slot nobody wrote then shows)."""
        self._engine._h.call("poison")

    def state(self, cache: int) -> torch.Tensor:
        s = self._engine._h.call("state", cache=cache)
        code = {"float32": 0, "bfloat16": 1, "int32": 2}[s["dtype"]]
        return wrap_device(s["address"], (s["rows"], s["row_elems"]), code)

    def bytes(self) -> int:
        return self._engine._h.call("counters")["cache_bytes"]


class _CacheView:
    """The engine's cache manager: the host-side allocator and the device arenas."""

    def __init__(self, engine: "Engine"):
        self._engine = engine
        self.alloc = BlockAllocator(_handle=core.Handle("allocator", engine._h.call("allocator")["handle"], keep=engine._h),
                                    _ids=engine.ids)
        self.layout = self.alloc.layout
        self.device_caches = _DeviceCachesView(engine)
        self.page_size = self.alloc.page_size
        self.max_requests = self.alloc.max_requests

    def kv_bytes_per_token(self) -> int:
        return self._engine._h.call("counters")["kv_bytes_per_token"]


def _ints(values) -> "ctypes.Array":
    return (ctypes.c_int * max(len(values), 1))(*values)


def _int_array(parts) -> np.ndarray:
    """The concatenation of integer sequences (lists or arrays) as one contiguous int32 array: for the
    token ids of a step, which may be thousands (a ctypes array built from a list costs ten times this)."""
    arrays = [np.asarray(p, dtype=np.int32).reshape(-1) for p in parts]
    if not arrays:
        return np.zeros(1, dtype=np.int32)
    out = arrays[0] if len(arrays) == 1 else np.concatenate(arrays)
    return np.ascontiguousarray(out) if out.size else np.zeros(1, dtype=np.int32)


class Engine:
    """A bound model, its cache and the step function over them."""

    def __init__(self, model: Model, *, max_tokens: int, page_size: int = 16, max_requests: int = 64,
                 max_step_tokens: int = 2048, use_cuda_graphs: bool = True, _handle: Optional[core.Handle] = None,
                 _ids: Optional[RequestIds] = None):
        self.model = model
        if _handle is None:
            _handle = core.Handle("engine", core.call(
                "global", None, "new_engine", model=model._handle_for_engine(), max_tokens=int(max_tokens), page_size=page_size,
                max_requests=max_requests, max_step_tokens=max_step_tokens, use_cuda_graphs=use_cuda_graphs)["handle"],
                keep=model._h)
        self._h = _handle
        self._lib = core.lib()
        self.ids = _ids or RequestIds()
        self.cache = _CacheView(self)
        self.vocab_size = model.spec.vocab_size
        c = self._h.call("counters")
        self.dtype = getattr(torch, c["dtype"])
        self.use_cuda_graphs = c["use_cuda_graphs"]

    # ---- counters (read from the library) ------------------------------------------------
    def _counter(name):
        return property(lambda self: self._h.call("counters")[name])

    steps_run = _counter("steps_run")
    graph_replays = _counter("graph_replays")
    stale_graphs = _counter("stale_graphs")
    burst_graphs_recorded = _counter("burst_graphs_recorded")
    recorded_graphs = _counter("recorded_graphs")
    h2d_bytes_total = _counter("h2d_bytes_total")
    d2h_bytes_total = _counter("d2h_bytes_total")
    last_h2d_bytes = _counter("last_h2d_bytes")
    last_launches = _counter("last_launches")
    del _counter

    # ---- request lifetime ------------------------------------------------------------
    def admit(self, rid: Hashable) -> int:
        return self._h.call("admit", rid=self.ids.of(rid))

    def release(self, rid: Hashable) -> None:
        self._h.call("release", rid=self.ids.of(rid))

    def length(self, rid: Hashable) -> int:
        return self._h.call("length", rid=self.ids.of(rid))

    def commit(self, rid: Hashable, new_len: int) -> None:
        """Advance a request's length after a burst (see decode_burst_async)."""
        self._h.call("commit", rid=self.ids.of(rid), new_len=int(new_len))

    # ---- running ------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], sampling: Optional[Sequence[SampleRow]] = None) -> torch.Tensor:
        """Run one step; returns float32 logits [wanted, vocab] on the device.  The tensor is the
        engine's workspace memory: the next step overwrites it.  With `sampling` (one SampleRow per
        wanted place) the drawn tokens are read with `read_sampled(n)` afterwards."""
        n = len(entries)
        rids = (ctypes.c_longlong * max(n, 1))(*[self.ids.of(e.rid) for e in entries])
        tokens = _int_array([e.tokens for e in entries])
        want = [int(w) for e in entries for w in e.want]
        samp = None
        if sampling is not None:
            flat = [v for r in sampling for v in (r.temperature, float(r.top_k), r.top_p, r.uniform)]
            samp = (ctypes.c_float * max(len(flat), 1))(*flat)
        logits, rows, cols = ctypes.c_void_p(), ctypes.c_int(), ctypes.c_int()
        code = self._lib.sandy_engine_step(ctypes.c_void_p(self._h.handle), n, rids, _ints([len(e.tokens) for e in entries]),
                                           tokens.ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
                                           _ints([len(e.want) for e in entries]), _ints(want), samp,
                                           ctypes.byref(logits), ctypes.byref(rows), ctypes.byref(cols))
        if code != 0:
            core.raise_last_error()
        self.synchronize()
        return wrap_device(logits.value, (rows.value, cols.value), 0)

    def read_sampled(self, n: int) -> List[int]:
        """The tokens drawn by the last step with `sampling`, on the host.  The step's status words
        come back in the same wait; a non-zero one raises (the tokens are not valid then)."""
        out = (ctypes.c_int * max(n, 1))()
        if self._lib.sandy_engine_read_sampled(ctypes.c_void_p(self._h.handle), n, out) != 0:
            core.raise_last_error()
        return list(out[:n])

    def decode_burst_async(self, entries: Sequence[StepEntry], sampling: Sequence[SampleRow], uniforms: np.ndarray,
                           in_flight: int = 0) -> BurstHandle:
        """Queue `n = uniforms.shape[0]` decode steps of the same requests back to back on the
        device.  Every entry brings one token and wants its logits; step j of request r is drawn
        with sampling[r] and the uniform number uniforms[j, r]; the token drawn in step j is the
        input of step j + 1.  Pages for all n steps are reserved before anything runs (OutOfPages
        otherwise, with nothing taken).  The requests' lengths are NOT advanced: the caller commits
        as many of each request's steps as it keeps.  With `in_flight` > 0 the burst continues one
        of the same requests, in the same order, that was queued before and is `in_flight` steps
        long; the entries' token ids are ignored then."""
        S = len(entries)
        u = np.ascontiguousarray(uniforms, dtype=np.float32)
        n = int(u.shape[0])
        rids = (ctypes.c_longlong * max(S, 1))(*[self.ids.of(e.rid) for e in entries])
        flat = [v for r in sampling for v in (r.temperature, float(r.top_k), r.top_p, 0.0)]
        burst = self._lib.sandy_engine_decode_burst_async(
            ctypes.c_void_p(self._h.handle), S, rids, _ints([int(e.tokens[0]) for e in entries]),
            (ctypes.c_float * max(len(flat), 1))(*flat), u.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), n, int(in_flight))
        if burst < 0:
            core.raise_last_error()
        return BurstHandle(n, S, burst)

    def decode_burst(self, entries, sampling, uniforms) -> np.ndarray:
        return self.burst_tokens(self.decode_burst_async(entries, sampling, uniforms))

    def burst_tokens(self, handle: BurstHandle) -> np.ndarray:
        """Wait for a burst queued by decode_burst_async; its tokens, int32 [n, requests]."""
        out = np.zeros((handle.n, handle.S), dtype=np.int32)
        if self._lib.sandy_engine_burst_tokens(ctypes.c_void_p(self._h.handle), handle.burst,
                                               out.ctypes.data_as(ctypes.POINTER(ctypes.c_int))) != 0:
            core.raise_last_error()
        return out

    def synchronize(self) -> None:
        if self._lib.sandy_engine_synchronize(ctypes.c_void_p(self._h.handle)) != 0:
            core.raise_last_error()

    def check_status(self) -> None:
        """Raise if a kernel reported bad input or an expired wait since the last check."""
        self._h.call("check_status")

    # ---- device timing on the engine's stream ---------------------------------------------
    def mark(self, which: int) -> None:
        if self._lib.sandy_engine_mark(ctypes.c_void_p(self._h.handle), which) != 0:
            core.raise_last_error()

    def hold(self, microseconds: int) -> None:
        """Keeps the engine's stream busy for so long (a kernel that only waits): what the host queues
        meanwhile runs back to back behind it.  For timing the device's share of a step."""
        if self._lib.sandy_engine_hold(ctypes.c_void_p(self._h.handle), int(microseconds)) != 0:
            core.raise_last_error()

    def elapsed_ms(self) -> float:
        ms = self._lib.sandy_engine_elapsed_ms(ctypes.c_void_p(self._h.handle))
        if ms < 0:
            core.raise_last_error()
        return float(ms)
