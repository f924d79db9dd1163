"""The scheduler: which requests run in the next step, with how many tokens each.

It works on the host-side BlockAllocator only, so all of its decisions can be tested without a GPU.
The decisions are the host library's (core/scheduler.cpp); this module is its Python face, used by
the tests and by callers that drive plan / complete themselves.  (Generation drives the library's
scheduler inside the library, see engine/llm.py.)

The reference lets exactly one request generate at a time (a FIFO ticket gate,
src/server/GenerationGate.cpp:13-37) and runs it to the end: the prompt in chunks of
`prefillChunkTokens` (default 2048, src/server/Session.h:23, loop :423-448), then token by token
(:477-514); finish reasons "stop" (the stop token is part of the output, :481-497) and "length"
(:498-501; max_tokens == 0 finishes at once with no forward, :407-417).  Those meanings are kept.
What is new here is that many requests are live at once:

  * admission: first come first served, while a state slot is free, fewer than `max_live` are
    running and the pool can hold the request's first portion;
  * a token budget per step: every running request that is decoding gets its one token first; what
    is left of the budget goes to prompts, oldest first, in portions of at most `prefill_chunk`
    tokens, cut wherever the budget or the free pages end;
  * pages run out: a decoding request that cannot get its next page preempts the most recently
    admitted running request (possibly itself): that request gives back all its pages and goes
    back to the head of the waiting queue with prompt + output so far, to be recomputed later.  A
    request that could never fit in the whole pool is refused when it is added.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Dict, Hashable, List, Optional

from .. import core
from ..cache.pages import BlockAllocator
from ..errors import RequestRefused  # noqa: F401  (re-exported)
from ..sampling.params import SamplingParams


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


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

    def _update(self, j: dict) -> None:
        self.state = RequestState(j["state"])
        self.output[:] = j["output"]
        self.computed, self.finish_reason = j["computed"], j["finish_reason"]
        self.preemptions, self.admitted_at = j["preemptions"], j["admitted_at"]


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
    plan: int = 0              # the library's handle on this plan

    @property
    def n_tokens(self) -> int:
        return sum(p.count for p in self.portions)


class Scheduler:
    def __init__(self, alloc: BlockAllocator, *, max_step_tokens: int = 2048, prefill_chunk: int = 2048,
                 max_live: int = 64, max_positions: Optional[int] = None):
        self.alloc = alloc
        self.max_step_tokens, self.prefill_chunk = max_step_tokens, prefill_chunk
        self.max_live, self.max_positions = max_live, max_positions
        self._h = core.Handle("scheduler", core.call(
            "global", None, "new_scheduler", allocator=alloc._h.handle, max_step_tokens=max_step_tokens,
            prefill_chunk=prefill_chunk, max_live=max_live, max_positions=max_positions)["handle"], keep=alloc._h)
        self._requests: Dict[int, Request] = {}

    def _sync(self) -> None:
        for i, r in self._requests.items():
            r._update(self._h.call("request", rid=i))

    def add(self, req: Request) -> None:
        i = self.alloc.ids.of(req.rid)
        j = self._h.call("add", rid=i, prompt=[int(t) for t in req.prompt], max_tokens=int(req.max_tokens),
                         stop_ids=sorted(int(s) for s in req.stop_ids))
        self._requests[i] = req
        req._update(j)

    def has_work(self) -> bool:
        return self._h.call("has_work")

    def plan(self) -> StepPlan:
        """Decide the next step and reserve its pages.  May preempt running requests."""
        j = self._h.call("plan")
        self._sync()
        return StepPlan([Portion(self._requests[p["rid"]], p["start"], p["count"], p["samples"]) for p in j["portions"]],
                        [self._requests[i] for i in j["preempted"]], j["plan"])

    def complete(self, plan: StepPlan, sampled: Dict[Hashable, int]) -> List[Request]:
        """The planned step ran.  `sampled[rid]` is the token drawn for every portion with `samples`.
        Returns the requests that finished."""
        done = self._h.call("complete", plan=plan.plan,
                            sampled={str(self.alloc.ids.of(rid)): int(t) for rid, t in sampled.items()})
        self._sync()
        return [self._requests[i] for i in done]

    def abort(self, rid: Hashable, reason: str = "cancelled") -> Optional[Request]:
        i = self._h.call("abort", rid=self.alloc.ids.of(rid), reason=reason)
        self._sync()
        return None if i is None else self._requests[i]

    @property
    def stats(self) -> Dict[str, int]:
        return self._h.call("stats")
