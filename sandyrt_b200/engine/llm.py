"""LLM: the Python entry point.  Model folder in, generated token ids out.

    llm = LLM("path/to/model", dtype="bfloat16")
    results = llm.generate([[15496, 11, 616, 1438, 318]], max_tokens=32)
    results[0].output_ids, results[0].finish_reason

The call mirrors the reference's Model::generate(requestId, inputIds, maxTokens,
stopTokenIds, samplingOverrides, control, onToken) -> GenerateResult
(src/server/Model.h:34-48) and its GenerateResult fields (src/server/Session.h:25-34):
output ids, finish reason, prompt and completion token counts, prefill and decode times
and rates.  Unlike the reference, which serves one request at a time behind a gate, all
requests given to `generate` (or added with `add_request`) run together under the scheduler.

Tokens go in and come out as host integers; every step copies its inputs to the device and
reads the drawn tokens back.
"""
from __future__ import annotations

import dataclasses
import sys
import time
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..models.model import Model, load_model
from ..sampling.params import SamplingParams
from ..sampling.sampler import fresh_seed, uniform_for
from .scheduler import Portion, Request, RequestRefused, RequestState, Scheduler, StepPlan
from ..cache.pages import OutOfPages
from .step import MAX_BURST, Engine, SampleRow, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


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


def _rate(tokens: int, ms: float) -> float:
    return tokens / (ms / 1000.0) if ms > 0 else 0.0


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
        if not torch.cuda.is_available():
            raise RuntimeError("sandyrt_b200 needs a CUDA device; there is no CPU path")
        if isinstance(model, Model):
            self.model = model
        else:
            self.model = load_model(model, device=device, dtype=_DTYPES[dtype])
        limit = self.model.max_positions
        if max_context_tokens and max_context_tokens > 0:
            limit = min(limit, max_context_tokens) if limit else max_context_tokens
        self.max_positions = limit
        if cache_tokens is None:
            cache_tokens = min(max_live * (limit or 4096), 1 << 20)
        self.engine = Engine(self.model, max_tokens=cache_tokens, page_size=page_size, max_requests=max_live,
                             max_step_tokens=max_step_tokens, use_cuda_graphs=use_cuda_graphs)
        self.scheduler = Scheduler(self.engine.cache.alloc, max_step_tokens=max_step_tokens,
                                   prefill_chunk=prefill_chunk_tokens, max_live=max_live,
                                   max_positions=limit, admit=self.engine.admit)
        self.eos_token_ids = frozenset(int(t) for t in (eos_token_ids or ()))
        self.max_burst = max(1, min(int(max_burst), MAX_BURST)) if self.engine.use_cuda_graphs else 1
        self.decode_steps_run = 0
        # A burst queued on the device whose tokens the host has not read yet: (handle, requests).
        # While one is in flight the next may be queued behind it (see _advance), so the device
        # does not wait for the host between bursts.
        self._inflight: Optional[Tuple[object, List[Request]]] = None
        self.pipeline_bursts = pipeline_bursts
        self.bursts_queued_ahead = 0
        self._requests: Dict[Hashable, Request] = {}
        self._seeds: Dict[Hashable, int] = {}
        self._next_id = 0

    # ---- request interface ----------------------------------------------------------------
    def add_request(self, prompt_ids: Sequence[int], *, max_tokens: int = 16,
                    sampling: Optional[SamplingParams] = None, stop_token_ids: Sequence[int] = (),
                    request_id: Optional[Hashable] = None) -> Hashable:
        sampling = (sampling or SamplingParams()).validate()
        rid = request_id if request_id is not None else f"req-{self._next_id}"
        self._next_id += 1
        if rid in self._requests:
            raise RequestRefused(f"request id {rid!r} is in use")
        vocab = self.model.spec.vocab_size
        prompt = [int(t) for t in prompt_ids]
        for t in prompt:
            if not (0 <= t < vocab):
                raise RequestRefused(f"token id {t} is outside the vocabulary of {vocab}")
        req = Request(rid, prompt, int(max_tokens), frozenset(int(s) for s in stop_token_ids) | self.eos_token_ids,
                      sampling)
        req.t_added = time.perf_counter()
        self.scheduler.add(req)
        self._requests[rid] = req
        self._seeds[rid] = sampling.seed if sampling.seed is not None else fresh_seed()
        return rid

    def has_work(self) -> bool:
        """Whether a call of `step` would do anything: a request is waiting or running, or a burst
        queued on the device has not been read yet."""
        return self.scheduler.has_work() or self._inflight is not None

    def finished(self, rid: Hashable) -> bool:
        return self._requests[rid].state is RequestState.FINISHED

    def _burst_length(self, plan: StepPlan) -> int:
        """How many decode steps may run on the device before the host looks again: more than
        one only when every request of the step is decoding and nobody waits to be admitted,
        and never past a request's token limit, the model's positions or the free pages."""
        if self.max_burst <= 1 or self.scheduler.waiting or not plan.portions:
            return 1
        for p in plan.portions:
            if p.count != 1 or not p.samples or not p.request.output:
                return 1
        return self._steps_possible([p.request for p in plan.portions], 0)

    def _steps_possible(self, reqs: Sequence[Request], in_flight: int) -> int:
        """Steps (at most max_burst, possibly 0) that all of `reqs` can still take when they are
        already `in_flight` steps ahead of what the host has seen: no request past its token limit
        or the model's positions, and pages for all of them."""
        n = self.max_burst
        for r in reqs:
            n = min(n, r.max_tokens - len(r.output) - in_flight)
            if self.max_positions is not None:
                n = min(n, self.max_positions - r.computed - in_flight)
        alloc = self.engine.cache.alloc
        while n > 1:
            need = [0] * len(alloc.pools)
            for r in reqs:
                for g, k in enumerate(alloc.pages_needed(r.rid, r.computed + in_flight + n)):
                    need[g] += k
            if all(k <= alloc.free_pages(g) for g, k in enumerate(need)):
                break
            n //= 2
        return max(n, 1 if in_flight == 0 else 0)

    def _queue_burst(self, reqs: List[Request], n: int, in_flight: int):
        """Queue n decode steps of `reqs` on the device (behind `in_flight` steps already queued)."""
        entries = [StepEntry(r.rid, [0 if in_flight else r.tokens[-1]], [0]) for r in reqs]
        rows, uniforms = [], np.zeros((n, len(reqs)), dtype=np.float32)
        for i, r in enumerate(reqs):
            sp = r.sampling
            rows.append(SampleRow(0.0 if sp.greedy else sp.temperature, sp.top_k, sp.top_p, 0.0))
            if not sp.greedy:
                for j in range(n):
                    uniforms[j, i] = uniform_for(self._seeds[r.rid], len(r.output) + in_flight + j)
        return self.engine.decode_burst_async(entries, rows, uniforms, in_flight=in_flight)

    def _collect_burst(self, handle, reqs: List[Request]) -> List[Tuple[Request, int]]:
        """Read a queued burst's tokens and do the scheduler's bookkeeping for each of its steps in
        order.  A request that finishes part of the way (or was finished or aborted while the
        burst ran) keeps only the tokens up to its finish; what the device computed for it after
        that is dropped."""
        tokens = self.engine.burst_tokens(handle)       # raises if a kernel of the burst reported a fault
        n = handle.n
        self.decode_steps_run += n
        now = time.perf_counter()
        got: List[Tuple[Request, int]] = []
        alive = [i for i, r in enumerate(reqs) if r.state is RequestState.RUNNING]
        if any(int(tokens[j, i]) < 0 for j in range(n) for i in alive):
            raise ValueError("sampling logits must not contain NaN")         # Sampler.cpp:64-67
        for j in range(n):
            if not alive:
                break
            sub = StepPlan([Portion(reqs[i], reqs[i].computed, 1, True) for i in alive], [])
            sampled = {reqs[i].rid: int(tokens[j, i]) for i in alive}
            got += [(reqs[i], int(tokens[j, i])) for i in alive]
            for r in self.scheduler.complete(sub, sampled):
                r.t_finished = now
            alive = [i for i in alive if reqs[i].state is RequestState.RUNNING]
        return got

    def _advance(self) -> List[Tuple[Request, int]]:
        """A burst is in flight.  If its requests can all go on (nobody is waiting to be admitted,
        nobody is known to have finished, tokens, positions and pages allow it), queue the next
        burst behind it BEFORE reading its tokens; then read them.  A request that turns out to
        have stopped inside the burst just read has wasted rows in the one queued behind it,
        nothing more: its pages are given back at once, but anything that could reuse them is
        queued on the same stream behind that burst."""
        handle, reqs = self._inflight
        nxt = None
        if self.pipeline_bursts and not self.scheduler.waiting \
                and all(r.state is RequestState.RUNNING for r in reqs):
            n = self._steps_possible(reqs, handle.n)
            if n >= 1:
                try:
                    nxt = self._queue_burst(reqs, n, handle.n)
                    self.bursts_queued_ahead += 1
                except OutOfPages:
                    nxt = None
        got = self._collect_burst(handle, reqs)
        self._inflight = (nxt, reqs) if nxt is not None else None
        return got

    def _step_burst(self, plan: StepPlan, n: int) -> List[Tuple[Request, int]]:
        """Queue n decode steps (Engine.decode_burst_async) and hand them to _advance, which may
        queue the following burst before it reads this one's tokens."""
        reqs = [p.request for p in plan.portions]
        self._inflight = (self._queue_burst(reqs, n, 0), reqs)
        return self._advance()

    def step(self) -> List[Tuple[Request, int]]:
        """Plan and run one step (or, when every request is decoding, a burst of steps on the
        device).  Returns (request, token) for every token drawn, in order."""
        if self._inflight is not None:
            return self._advance()
        plan = self.scheduler.plan()
        if not plan.portions:
            return []
        n_burst = self._burst_length(plan)
        if n_burst > 1:
            return self._step_burst(plan, n_burst)
        now = time.perf_counter()
        entries, sampled_reqs = [], []
        for p in plan.portions:
            req = p.request
            if req.t_first_scheduled == 0.0:
                req.t_first_scheduled = now
            toks = req.tokens[p.start:p.start + p.count]
            entries.append(StepEntry(req.rid, toks, [p.count - 1] if p.samples else []))
            if p.samples:
                sampled_reqs.append(req)
        rows = []
        for r in sampled_reqs:
            sp = r.sampling
            rows.append(SampleRow(0.0 if sp.greedy else sp.temperature, sp.top_k, sp.top_p,
                                  0.0 if sp.greedy else uniform_for(self._seeds[r.rid], len(r.output))))
        self.engine.step(entries, sampling=rows)
        sampled: Dict[Hashable, int] = {}
        if sampled_reqs:
            n = len(sampled_reqs)
            host = self.engine.read_sampled(n)          # raises if a kernel of the step reported a fault
            if any(t < 0 for t in host):
                raise ValueError("sampling logits must not contain NaN")     # Sampler.cpp:64-67
            sampled = {r.rid: t for r, t in zip(sampled_reqs, host)}
        now = time.perf_counter()
        for r in sampled_reqs:
            if r.t_first_token == 0.0:
                r.t_first_token = now
        for r in self.scheduler.complete(plan, sampled):
            r.t_finished = now
        self.decode_steps_run += 1
        return [(r, sampled[r.rid]) for r in sampled_reqs]

    def result(self, rid: Hashable) -> GenerateResult:
        r = self._requests[rid]
        t_end = r.t_finished or time.perf_counter()
        prefill_ms = max(0.0, ((r.t_first_token or t_end) - (r.t_first_scheduled or r.t_added)) * 1e3)
        decode_ms = max(0.0, (t_end - (r.t_first_token or t_end)) * 1e3)
        n_out = len(r.output)
        return GenerateResult(list(r.output), r.finish_reason or "", len(r.prompt), n_out, prefill_ms, decode_ms,
                              _rate(len(r.prompt), prefill_ms), _rate(max(n_out - 1, 0), decode_ms), r.preemptions)

    def forget(self, rid: Hashable) -> None:
        self._requests.pop(rid, None)
        self._seeds.pop(rid, None)

    def abort(self, rid: Hashable) -> None:
        self.scheduler.abort(rid, "cancelled")

    def drain(self) -> List[Tuple[Request, int]]:
        """Read the bursts still queued on the device (and do their bookkeeping) without queueing
        anything new.  Returns the tokens they drew for requests that were still running."""
        got: List[Tuple[Request, int]] = []
        while self._inflight is not None:
            handle, reqs = self._inflight
            self._inflight = None
            got += self._collect_burst(handle, reqs)
        return got

    # ---- the blocking convenience -----------------------------------------------------------
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], *, max_tokens: int = 16,
                 temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, seed: Optional[int] = None,
                 stop_token_ids: Sequence[int] = (),
                 on_token: Optional[Callable[[Hashable, int], bool]] = None,
                 report: bool = False) -> List[GenerateResult]:
        """Generate for one prompt (a list of ids) or several (a list of lists).  `on_token`
        is called with (request index, token) for every new token; returning False cancels
        that request (finish reason "cancelled"; the reference fails the request with
        "request cancelled", src/server/Session.cpp:491-492)."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        batch = [prompts] if single else list(prompts)
        rids = []
        for i, p in enumerate(batch):
            s = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p,
                               seed=None if seed is None else seed + i)
            rids.append(self.add_request(p, max_tokens=max_tokens, sampling=s, stop_token_ids=stop_token_ids))
        index = {rid: i for i, rid in enumerate(rids)}
        cancelled = set()
        delivered = {rid: 0 for rid in rids}
        while any(self._requests[r].state is not RequestState.FINISHED for r in rids):
            got = self.step()
            if on_token:
                for r, token in got:
                    if r.rid not in index or r.rid in cancelled:
                        continue
                    delivered[r.rid] += 1
                    if on_token(index[r.rid], token) is False:
                        # the request ends with the token just delivered; what a burst had
                        # already drawn beyond it is dropped
                        cancelled.add(r.rid)
                        if r.state is not RequestState.FINISHED:
                            self.abort(r.rid)
                        del r.output[delivered[r.rid]:]
                        r.finish_reason = "cancelled"
        results = [self.result(r) for r in rids]
        for r in rids:
            self.forget(r)
        if report:
            for res in results:
                # the reference prints the same line to stderr (src/server/Session.cpp:539-548)
                print(f"sandy throughput: prefill_tokens={res.prompt_tokens} prefill_ms={res.prefill_ms:.3f} "
                      f"prefill_toks_per_s={res.prefill_tokens_per_second:.3f} "
                      f"decode_tokens={res.completion_tokens} decode_ms={res.decode_ms:.3f} "
                      f"decode_toks_per_s={res.decode_tokens_per_second:.3f}", file=sys.stderr)
        return results
