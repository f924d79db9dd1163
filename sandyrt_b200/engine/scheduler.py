"""The scheduler: which requests run in the next step, with how many tokens each.

It works on the host-side BlockAllocator only, so all of its decisions can be tested
without a GPU.

The reference lets exactly one request generate at a time (a FIFO ticket gate,
src/server/GenerationGate.cpp:13-37) and runs it to the end: the prompt in chunks of
`prefillChunkTokens` (default 2048, src/server/Session.h:23, loop :423-448), then token by
token (:477-514); finish reasons "stop" (the stop token is part of the output, :481-497)
and "length" (:498-501; max_tokens == 0 finishes at once with no forward, :407-417).
Those meanings are kept.  What is new here is that many requests are live at once:

  * admission: first come first served, while a state slot is free, fewer than
    `max_live` are running and the pool can hold the request's first portion;
  * a token budget per step: every running request that is decoding gets its one token
    first; what is left of the budget goes to prompts, oldest first, in portions of at
    most `prefill_chunk` tokens, cut wherever the budget or the free pages end;
  * pages run out: a decoding request that cannot get its next page preempts the most
    recently admitted running request (possibly itself): that request gives back all its
    pages and goes back to the head of the waiting queue with prompt + output so far, to
    be recomputed later.  A request that could never fit in the whole pool is refused
    when it is added.
"""
from __future__ import annotations

import collections
import dataclasses
import enum
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.pages import BlockAllocator, NoFreeSlot, OutOfPages
from ..sampling.params import SamplingParams


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class RequestRefused(ValueError):
    """The request can never be served (empty prompt, too long for the model or the pool)."""


@dataclasses.dataclass(eq=False)
class Request:
    rid: Hashable
    prompt: List[int]
    max_tokens: int
    stop_ids: frozenset = frozenset()
    sampling: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    output: List[int] = dataclasses.field(default_factory=list)
    state: RequestState = RequestState.WAITING
    computed: int = 0                  # tokens of prompt+output whose keys/values are cached
    finish_reason: Optional[str] = None
    preemptions: int = 0
    admitted_at: int = -1              # admission counter value (larger = admitted later)
    # timing, filled by the caller of the scheduler
    t_added: float = 0.0
    t_first_scheduled: float = 0.0
    t_first_token: float = 0.0
    t_finished: float = 0.0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def pending(self) -> int:
        """Tokens not yet run through the model."""
        return self.n_tokens - self.computed


@dataclasses.dataclass
class Portion:
    """One request's share of a planned step."""
    request: Request
    start: int                 # index into request.tokens of the first token run
    count: int
    samples: bool              # the portion reaches the request's last token: sample after it


@dataclasses.dataclass
class StepPlan:
    portions: List[Portion]
    preempted: List[Request]

    @property
    def n_tokens(self) -> int:
        return sum(p.count for p in self.portions)


class Scheduler:
    def __init__(self, alloc: BlockAllocator, *, max_step_tokens: int = 2048, prefill_chunk: int = 2048,
                 max_live: int = 64, max_positions: Optional[int] = None, admit=None):
        """admit: how a request takes its state slot (default: the allocator's own `admit`).  The
        entry point passes the cache manager's, which also zeroes the slot's fixed-size state on
        the device, so that a request never starts from the state of the slot's last holder."""
        if max_step_tokens <= 0 or prefill_chunk <= 0 or max_live <= 0:
            raise ValueError("token budget, chunk size and request limit must be positive")
        self.alloc = alloc
        self._admit = admit if admit is not None else alloc.admit
        self.max_step_tokens = max_step_tokens
        self.prefill_chunk = prefill_chunk
        self.max_live = max_live
        self.max_positions = max_positions
        self.waiting: Deque[Request] = collections.deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._admissions = 0
        self.stats = collections.Counter()

    # ---- adding -------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise RequestRefused("the prompt must not be empty")      # Session.cpp:389-390
        if req.max_tokens < 0:
            raise RequestRefused("max_tokens must be >= 0")           # Session.cpp:391-392
        if self.max_positions is not None and len(req.prompt) > self.max_positions:
            raise RequestRefused(f"the prompt has {len(req.prompt)} tokens, the model has "
                                 f"{self.max_positions} positions")
        longest = len(req.prompt) + max(req.max_tokens - 1, 0)
        if self.max_positions is not None:
            longest = min(longest, self.max_positions)
        for g, pool in enumerate(self.alloc.pools):
            need = self._pages_for(g, longest)
            if need > pool.num_pages:
                raise RequestRefused(f"the request may grow to {longest} tokens, which needs {need} pages "
                                     f"of cache group {g}; the pool has {pool.num_pages}")
        if req.max_tokens == 0:
            req.state, req.finish_reason = RequestState.FINISHED, "length"
            self.finished.append(req)
            return
        req.state = RequestState.WAITING
        self.waiting.append(req)

    def _pages_for(self, group: int, n_tokens: int) -> int:
        """Most pages of `group` a request of n_tokens holds at one time."""
        ps = self.alloc.page_size
        window = self.alloc.layout.groups[group].spec.window
        if window:
            # pages covering the window plus the portion being appended
            span = min(n_tokens, window + self.prefill_chunk)
            return min(-(-n_tokens // ps), -(-span // ps) + 1)
        return -(-n_tokens // ps)

    # ---- planning -------------------------------------------------------------------------
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self.alloc.release(req.rid)
        self.running.remove(req)
        req.state = RequestState.WAITING
        req.computed = 0
        req.preemptions += 1
        self.waiting.appendleft(req)
        plan.preempted.append(req)
        plan.portions = [p for p in plan.portions if p.request is not req]
        self.stats["preemptions"] += 1

    def _fit(self, req: Request, want: int) -> int:
        """Largest n <= want such that pages for req.computed + n tokens can be reserved."""
        lo = req.computed
        needed = self.alloc.pages_needed(req.rid, lo + want)
        if all(n <= self.alloc.free_pages(g) for g, n in enumerate(needed)):
            return want
        ps = self.alloc.page_size
        best = want
        for g, pool in enumerate(self.alloc.pools):
            have_blocks = len(self.alloc.block_list(req.rid, g))
            room = (have_blocks + pool.free_pages) * ps - lo
            best = min(best, room)
        return max(best, 0)

    def plan(self) -> StepPlan:
        """Decide the next step and reserve its pages.  May preempt running requests."""
        plan = StepPlan([], [])
        budget = self.max_step_tokens

        # 1. running requests that are decoding: one token each, oldest first
        for req in sorted(self.running, key=lambda r: r.admitted_at):
            if req.state is not RequestState.RUNNING or req.pending != 1 or not req.output:
                continue
            if budget <= 0:
                break
            while req.state is RequestState.RUNNING and not self.alloc.can_reserve(req.rid, req.computed + 1):
                victim = max(self.running, key=lambda r: r.admitted_at)
                self._preempt(victim, plan)
            if req.state is not RequestState.RUNNING:
                continue                    # it preempted itself
            self.alloc.reserve(req.rid, req.computed + 1)
            plan.portions.append(Portion(req, req.computed, 1, True))
            budget -= 1

        # 2. running requests still working through their prompt (or a recomputation)
        scheduled = {id(p.request) for p in plan.portions}
        for req in sorted(self.running, key=lambda r: r.admitted_at):
            if id(req) in scheduled or budget <= 0:
                continue
            n = self._fit(req, min(req.pending, self.prefill_chunk, budget))
            if n <= 0:
                continue
            self.alloc.reserve(req.rid, req.computed + n)
            plan.portions.append(Portion(req, req.computed, n, n == req.pending))
            budget -= n

        # 3. admit waiting requests, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.max_live:
            req = self.waiting[0]
            if any(req is r for r in plan.preempted):
                break                       # never re-admit in the step that preempted it
            if self.alloc.free_slots() == 0:
                break
            first = min(req.pending, self.prefill_chunk, budget)
            needed = self.alloc.pages_for_new_request(first)
            if any(n > self.alloc.free_pages(g) for g, n in enumerate(needed)):
                break
            self.waiting.popleft()
            self._admit(req.rid)
            self.alloc.reserve(req.rid, first)
            req.state = RequestState.RUNNING
            req.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(req)
            plan.portions.append(Portion(req, 0, first, first == req.pending))
            budget -= first
            self.stats["admissions"] += 1

        # 4. nothing could move although requests are live: every running request is in the
        #    middle of its prompt and the pool is full.  Give the newest one's pages to the rest.
        if not plan.portions and self.running:
            victim = max(self.running, key=lambda r: r.admitted_at)
            self._preempt(victim, plan)
            if self.running or self.waiting:
                again = self.plan()
                again.preempted = plan.preempted + again.preempted
                return again
        self.stats["steps"] += 1
        self.stats["tokens"] += plan.n_tokens
        return plan

    # ---- after the step ---------------------------------------------------------------------
    def complete(self, plan: StepPlan, sampled: Dict[Hashable, int]) -> List[Request]:
        """The planned step ran.  `sampled[rid]` is the token drawn for every portion with
        `samples`.  Returns the requests that finished."""
        done: List[Request] = []
        for p in plan.portions:
            req = p.request
            req.computed = p.start + p.count
            self.alloc.commit(req.rid, req.computed)
            if not p.samples:
                continue
            token = int(sampled[req.rid])
            req.output.append(token)
            reason = None
            if token in req.stop_ids:
                reason = "stop"
            elif len(req.output) >= req.max_tokens:
                reason = "length"
            elif self.max_positions is not None and req.n_tokens > self.max_positions:
                reason = "length"           # the new token has no position left to run at
            if reason:
                self._finish(req, reason)
                done.append(req)
        return done

    def _finish(self, req: Request, reason: str) -> None:
        req.state, req.finish_reason = RequestState.FINISHED, reason
        if req in self.running:
            self.running.remove(req)
            self.alloc.release(req.rid)
        self.finished.append(req)

    def abort(self, rid: Hashable, reason: str = "cancelled") -> Optional[Request]:
        for req in list(self.running):
            if req.rid == rid:
                self._finish(req, reason)
                return req
        for req in list(self.waiting):
            if req.rid == rid:
                self.waiting.remove(req)
                req.state, req.finish_reason = RequestState.FINISHED, reason
                self.finished.append(req)
                return req
        return None
