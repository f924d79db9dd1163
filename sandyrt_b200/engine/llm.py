"""LLM: the Python entry point.  Model folder in, generated token ids out.

    llm = LLM("path/to/model", dtype="bfloat16")
    results = llm.generate([[15496, 11, 616, 1438, 318]], max_tokens=32)
    results[0].output_ids, results[0].finish_reason

It is a thin face of the host library's LLM (core/llm.cpp: scheduler, step function, bursts of
decode steps queued ahead of the host).  The call mirrors the reference's
Model::generate(requestId, inputIds, maxTokens, stopTokenIds, samplingOverrides, control, onToken)
-> GenerateResult (src/server/Model.h:34-48) and its GenerateResult fields
(src/server/Session.h:25-34): output ids, finish reason, prompt and completion token counts,
prefill and decode times and rates.  Unlike the reference, which serves one request at a time
behind a gate, all requests given to `generate` (or added with `add_request`) run together under
the scheduler.

Tokens go in and come out as host integers; every step copies its inputs to the device and reads
the drawn tokens back.
"""
from __future__ import annotations

import ctypes

import numpy as np
import dataclasses
import json
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple, Union

from .. import core
from ..cache.pages import RequestIds
from ..errors import RequestRefused  # noqa: F401  (re-exported)
from ..models.model import Model, _device_index, load_model
from ..sampling.params import SamplingParams
from .step import MAX_BURST, Engine

_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclasses.dataclass
class GenerateResult:
    """Fields of the reference's GenerateResult (src/server/Session.h:25-34)."""
    output_ids: List[int]
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    prefill_tokens_per_second: float = 0.0
    decode_tokens_per_second: float = 0.0
    preemptions: int = 0


class _SchedulerView:
    def __init__(self, llm: "LLM"):
        self._llm = llm

    @property
    def stats(self) -> Dict[str, int]:
        return self._llm._h.call("scheduler_stats")

    @property
    def waiting(self) -> int:
        return self._llm._h.call("info")["n_waiting"]


class LLM:
    def __init__(self, model: Union[str, Model], *, dtype: str = "bfloat16", device: str = "cuda:0",
                 cache_tokens: Optional[int] = None, page_size: int = 16, max_live: int = 64,
                 max_step_tokens: int = 2048, prefill_chunk_tokens: int = 2048,
                 eos_token_ids: Optional[Sequence[int]] = None, max_context_tokens: int = 0,
                 use_cuda_graphs: bool = True, max_burst: int = 8, pipeline_bursts: bool = True):
        """cache_tokens: how many tokens the cache pool holds (default: room for `max_live`
        requests of full length, capped at 1M tokens).  eos_token_ids: stop tokens added to
        every request (default: the config's eos_token_id is NOT added; pass it to stop there).
        max_context_tokens: if > 0, a lower limit on a request's length than the model's.
        max_burst: most decode steps run on the device between two looks of the host (1 = the
        host sees every token as it is drawn; more = fewer round trips, tokens arrive in groups,
        and up to max_burst - 1 steps of a request that has just hit a stop token are wasted).
        pipeline_bursts: queue the next burst on the device before the tokens of the last one
        have been read (a request that stops is then noticed one burst later, its extra rows are
        wasted work; the tokens delivered are the same)."""
        self._lib = core.lib()
        if isinstance(model, Model):
            self.model = model
        else:
            import torch
            self.model = load_model(model, device=device, dtype=getattr(torch, _DTYPES[dtype]))
        opts = dict(dtype=_DTYPES[dtype], device=_device_index(device), cache_tokens=int(cache_tokens or 0),
                    page_size=page_size, max_live=max_live, max_step_tokens=max_step_tokens,
                    prefill_chunk_tokens=prefill_chunk_tokens, eos_token_ids=[int(t) for t in (eos_token_ids or ())],
                    max_context_tokens=max_context_tokens, use_cuda_graphs=use_cuda_graphs, max_burst=max_burst,
                    pipeline_bursts=pipeline_bursts)
        h = self._lib.sandy_llm_from_model(ctypes.c_void_p(self.model._handle_for_engine()), json.dumps(opts).encode())
        if not h:
            core.raise_last_error()
        self._h = core.Handle("llm", h)              # the library's LLM now owns the model
        self.model._moved_into(self._h)               # (the emptied model handle is given back as it goes away)
        self.ids = RequestIds()
        self._next_id = 0
        self._rid_of: Dict[int, Hashable] = {}       # library request id -> caller's id
        self._lib_id: Dict[Hashable, int] = {}
        eng = self._lib.sandy_llm_engine(ctypes.c_void_p(h))
        self.engine = Engine(self.model, max_tokens=0, _handle=core.Handle("engine", eng, owned=False, keep=self._h),
                             _ids=_LLMIds(self))
        self.scheduler = _SchedulerView(self)
        info = self._h.call("info")
        self.max_burst = info["max_burst"]
        self.pipeline_bursts = info["pipeline_bursts"]
        cap = max(max_live, 1) * MAX_BURST
        self._rids_buf = (ctypes.c_longlong * cap)()
        self._tok_buf = (ctypes.c_int * cap)()
        self._cap = cap

    decode_steps_run = property(lambda self: self._h.call("info")["decode_steps_run"])
    bursts_queued_ahead = property(lambda self: self._h.call("info")["bursts_queued_ahead"])

    # ---- request interface ----------------------------------------------------------------
    def add_request(self, prompt_ids: Sequence[int], *, max_tokens: int = 16, sampling: Optional[SamplingParams] = None,
                    stop_token_ids: Sequence[int] = (), request_id: Optional[Hashable] = None) -> Hashable:
        sp = sampling or SamplingParams()
        rid = request_id if request_id is not None else f"req-{self._next_id}"
        self._next_id += 1
        if rid in self._lib_id:
            raise RequestRefused(f"request id {rid!r} is in use")
        prompt = np.ascontiguousarray(np.asarray(prompt_ids, dtype=np.int64).reshape(-1).astype(np.int32))
        n_prompt = int(prompt.size)
        if n_prompt == 0:
            prompt = np.zeros(1, dtype=np.int32)
        stop = [int(s) for s in stop_token_ids]
        i = self._lib.sandy_llm_add_request(
            ctypes.c_void_p(self._h.handle), prompt.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), n_prompt, int(max_tokens),
            ctypes.c_float(sp.temperature), int(sp.top_k), ctypes.c_float(sp.top_p), 0 if sp.seed is None else 1,
            ctypes.c_ulonglong((sp.seed or 0) & ((1 << 64) - 1)), (ctypes.c_int * max(len(stop), 1))(*stop), len(stop))
        if i < 0:
            core.raise_last_error()
        self._rid_of[i] = rid
        self._lib_id[rid] = i
        return rid

    def has_work(self) -> bool:
        """Whether a call of `step` would do anything: a request is waiting or running, or a burst
        queued on the device has not been read yet."""
        return bool(self._lib.sandy_llm_has_work(ctypes.c_void_p(self._h.handle)))

    def finished(self, rid: Hashable) -> bool:
        r = self._lib.sandy_llm_finished(ctypes.c_void_p(self._h.handle), ctypes.c_longlong(self._lib_id[rid]))
        if r < 0:
            core.raise_last_error()
        return bool(r)

    def _pairs(self, n: int) -> List[Tuple[Hashable, int]]:
        if n < 0:
            core.raise_last_error()
        return [(self._rid_of[self._rids_buf[k]], self._tok_buf[k]) for k in range(min(n, self._cap))]

    def step(self) -> List[Tuple[Hashable, int]]:
        """Plan and run one step (or, when every request is decoding, a burst of steps on the
        device).  Returns (request id, token) for every token drawn, in order."""
        return self._pairs(self._lib.sandy_llm_step(ctypes.c_void_p(self._h.handle), self._rids_buf, self._tok_buf, self._cap))

    def drain(self) -> List[Tuple[Hashable, int]]:
        """Read the bursts still queued on the device (and do their bookkeeping) without queueing
        anything new.  Returns the tokens they drew for requests that were still running."""
        return self._pairs(self._lib.sandy_llm_drain(ctypes.c_void_p(self._h.handle), self._rids_buf, self._tok_buf, self._cap))

    def result(self, rid: Hashable) -> GenerateResult:
        return GenerateResult(**self._h.call("result", rid=self._lib_id[rid]))

    def output_ids(self, rid: Hashable) -> List[int]:
        return self._h.call("request", rid=self._lib_id[rid])["output"]

    def forget(self, rid: Hashable) -> None:
        i = self._lib_id.pop(rid, None)
        if i is not None:
            self._rid_of.pop(i, None)
            self._h.call("forget", rid=i)

    def abort(self, rid: Hashable) -> None:
        self._h.call("abort", rid=self._lib_id[rid])

    # ---- the blocking convenience -----------------------------------------------------------
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], *, max_tokens: int = 16,
                 temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, seed: Optional[int] = None,
                 stop_token_ids: Sequence[int] = (), on_token: Optional[Callable[[int, int], bool]] = None,
                 report: bool = False) -> List[GenerateResult]:
        """Generate for one prompt (a list of ids) or several (a list of lists).  `on_token` is
        called with (request index, token) for every new token; returning False cancels that
        request (finish reason "cancelled"; the reference fails the request with "request
        cancelled", src/server/Session.cpp:491-492)."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        batch = [list(prompts)] if single else [list(p) for p in prompts]
        flat = [int(t) for p in batch for t in p]
        lens = [len(p) for p in batch]
        params = dict(max_tokens=int(max_tokens), temperature=float(temperature), top_p=float(top_p), top_k=int(top_k),
                      seed=seed, stop_token_ids=[int(s) for s in stop_token_ids], report=bool(report))
        cb = None
        raised: List[BaseException] = []
        if on_token is not None:
            def _cb(_user, index, token):
                try:
                    return 0 if on_token(index, token) is False else 1
                except BaseException as e:        # stop the request; the exception is raised after the call
                    raised.append(e)
                    return 0
            cb = core.TOKEN_FN(_cb)
        out = self._lib.sandy_llm_generate(ctypes.c_void_p(self._h.handle), (ctypes.c_int * max(len(flat), 1))(*flat),
                                           (ctypes.c_int * max(len(lens), 1))(*lens), len(batch), json.dumps(params).encode(),
                                           cb, None)
        if raised:
            raise raised[0]
        if out is None:
            core.raise_last_error()
        return [GenerateResult(**r) for r in json.loads(out)]


class _LLMIds:
    """Request ids of the engine behind an LLM: the caller's ids of requests added through the LLM,
    and ids of its own for requests stepped directly through `llm.engine`."""

    def __init__(self, llm: LLM):
        self._llm = llm
        self._own = RequestIds()
        self._own._next = 1 << 40          # apart from the library's own numbering of added requests

    def of(self, rid: Hashable) -> int:
        i = self._llm._lib_id.get(rid)
        return i if i is not None else self._own.of(rid)

    def rid(self, i: int) -> Hashable:
        return self._llm._rid_of[i] if i in self._llm._rid_of else self._own.rid(i)

    def known(self, rid: Hashable) -> bool:
        return rid in self._llm._lib_id or self._own.known(rid)
