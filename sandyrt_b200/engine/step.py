"""The step function: one batch of (request, its next tokens) through the model.

`Engine.step(entries)` takes, for each request of the step, the tokens that follow what
the request already has in the cache (a portion of a prompt of any length, or one decoded
token) and the places among them whose logits are wanted.  It runs exactly those tokens as
one batch, reading everything earlier from the cache, appends their keys and values to the
cache, and returns float32 logits [wanted, vocab] in the order of the entries and of their
wanted places.  With `sampling` it also draws one token per wanted row on the device.

The reference's counterpart, Engine::runValues on one of two compiled graphs (decode with
input_id [1,1], prefill with input_id [1,n]; src/engine/Engine.h:100-104,
src/server/Model.cpp:216-255, inputs built in src/server/Session.cpp:167-206), serves one
request per call, returns logits for every row and samples on the host.  Here there is one
code path for every mix of requests, and rows nobody asked for are never computed past the
last layer.

All the step's index arrays (token ids, positions, request of each token, block tables,
wanted rows, sampling options) are packed on the host into one pinned buffer and reach the
device with one copy.  Steps in which every request brings a single token (decoding) are
captured as CUDA graphs, one per (requests, wanted rows, block-table width), and replayed:
the arrays live at fixed device addresses, so a replay only needs the copy before it.

`Engine.decode_burst` runs several decode steps of the same requests with no trip to the host
in between: the sampler writes each drawn token over the step's input token and moves the
position on, so the same recorded graph is simply replayed n times; pages for all n steps are
reserved beforehand and the drawn tokens of all steps come back in one copy.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import FREED, OutOfPages
from ..csrc import ops
from ..models.model import Model
from ..parts.base import StepContext, Workspace

MAX_BURST = 32      # most decode steps one decode_burst may run
MAX_GRAPHS = 64     # most recorded step shapes kept at a time


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


class StepError(Exception):
    pass


class _Staging:
    """A ring of pinned host buffers and ONE device buffer for the step's index arrays.  The
    device buffer keeps its address for the engine's lifetime unless a step outgrows it."""

    def __init__(self, device, capacity: int, depth: int = 4):
        self.device = device
        self.depth = depth
        self.turn = 0
        self.generation = 0
        self._allocate(capacity)

    def _allocate(self, capacity: int) -> None:
        self.capacity = capacity
        self.host = [torch.empty(capacity, dtype=torch.int32, pin_memory=True) for _ in range(self.depth)]
        self.host_np = [h.numpy() for h in self.host]
        self.events: List[Optional[torch.cuda.Event]] = [None] * self.depth
        self.dev = torch.empty(capacity, dtype=torch.int32, device=self.device)
        self.generation += 1

    def acquire(self, n: int) -> int:
        if n > self.capacity:
            self._allocate(1 << (n - 1).bit_length())
        i = self.turn
        self.turn = (self.turn + 1) % self.depth
        if self.events[i] is not None:
            self.events[i].synchronize()      # the copy that last used this buffer is done
        return i

    def send(self, i: int, n: int, start: int = 0) -> None:
        """Copy elements [start, n) of host buffer i to the same place of the device buffer."""
        self.dev[start:n].copy_(self.host[i][start:n], non_blocking=True)
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()


@dataclasses.dataclass
class _Prepared:
    ctx: StepContext
    sample: Optional[torch.Tensor]          # [temperature R | top_k R | top_p R | uniform R] (one step)
    key: Optional[Tuple]                    # graph key, None for steps that are not recorded
    burst: Optional[Tuple[torch.Tensor, torch.Tensor]] = None    # (uniform [n, R], row_step [R]) of a burst


@dataclasses.dataclass
class BurstHandle:
    """A burst of decode steps queued on the device (Engine.decode_burst_async)."""
    n: int                       # steps
    S: int                       # requests
    host: torch.Tensor           # pinned int32 buffer the tokens are copied to; the two status words follow them
    done: torch.cuda.Event       # recorded behind that copy


class Engine:
    """A bound model, its cache and the step function over them."""

    def __init__(self, model: Model, *, max_tokens: int, page_size: int = 16, max_requests: int = 64,
                 max_step_tokens: int = 2048, use_cuda_graphs: bool = True):
        if model.device is None:
            raise StepError("the model has no weights bound")
        if model.device.type != "cuda":
            raise StepError("the engine runs on a CUDA device only; there is no CPU path")
        self.model = model
        self.device = model.device
        self.dtype = model.compute_dtype
        self.vocab_size = model.spec.vocab_size
        self.cache = CacheManager(model.cache_specs(), page_size=page_size, max_tokens=max_tokens,
                                  max_requests=max_requests, device=self.device, dtype=self.dtype)
        self.workspace = Workspace(self.device)
        blocks_cap = -(-(-(-(model.max_positions or max_tokens) // page_size) + 8) // 32) * 32
        cap = 4 * max_step_tokens + 3 * max_requests + 1 + (5 + MAX_BURST) * max_requests \
            + len(self.cache.layout.groups) * max_requests * blocks_cap
        self._staging = _Staging(self.device, 1 << (cap - 1).bit_length())
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._sampled = torch.zeros(max(max_requests, 1), dtype=torch.int32, device=self.device)
        self._burst_tokens = torch.zeros(MAX_BURST * max(max_requests, 1), dtype=torch.int32, device=self.device)
        # two pinned buffers: the tokens of one burst are read while the next one runs
        self._burst_hosts = [torch.zeros(MAX_BURST * max(max_requests, 1) + 2, dtype=torch.int32, pin_memory=True)
                             for _ in range(2)]
        self._token_host = torch.zeros(max(max_requests, 1) + 2, dtype=torch.int32, pin_memory=True)
        self._burst_turn = 0
        self._burst_flip = 0
        self.use_cuda_graphs = use_cuda_graphs and model.graph_safe
        self._graphs: Dict[Tuple, Tuple] = {}
        self._seen: Dict[Tuple, int] = {}
        self._table_rows: Dict[Tuple[Hashable, int], Tuple[int, np.ndarray]] = {}
        self.steps_run = 0
        self.graph_replays = 0
        self.stale_graphs = 0
        self.burst_graphs_recorded = 0   # whole bursts recorded as one graph so far
        self.last_h2d_bytes = 0
        self.h2d_bytes_total = 0         # bytes of step arrays copied to the device so far
        self.d2h_bytes_total = 0         # bytes of drawn tokens copied back so far (bursts; the entry point adds its own)
        self.last_launches = 0

    # ---- request lifetime ------------------------------------------------------------
    def admit(self, rid: Hashable) -> int:
        return self.cache.admit(rid)

    def release(self, rid: Hashable) -> None:
        self.cache.release(rid)
        for g in self.cache.layout.groups:
            self._table_rows.pop((rid, g.index), None)

    def length(self, rid: Hashable) -> int:
        return self.cache.alloc.length(rid)

    # ---- packing a step ----------------------------------------------------------------
    def _table_row(self, rid: Hashable, group: int) -> np.ndarray:
        """A request's block list as an int32 array, rebuilt only when the list has changed
        (a page was added, or a window gave pages back)."""
        stamp = self.cache.alloc.block_version(rid)
        hit = self._table_rows.get((rid, group))
        if hit is None or hit[0] != stamp:
            hit = (stamp, np.asarray(self.cache.alloc.block_list(rid, group), dtype=np.int32))
            self._table_rows[(rid, group)] = hit
            if len(self._table_rows) > 4 * self.cache.max_requests * max(1, len(self.cache.layout.groups)):
                live = self.cache.alloc
                self._table_rows = {k: v for k, v in self._table_rows.items() if k[0] in live}
        return hit[1]

    def _prepare(self, entries: Sequence[StepEntry], sampling: Optional[Sequence[SampleRow]],
                 burst_uniform: Optional[np.ndarray] = None, in_flight: int = 0) -> _Prepared:
        """Check the entries, reserve pages, pack the step's arrays and copy them to the device.
        burst_uniform: float32 [n_steps, R] for a burst of n_steps decode steps.
        in_flight: this burst continues one of the same requests that is still running on the
        device, `in_flight` steps long: every request is that many tokens further than its
        committed length, and its next token is already where the sampler left it, so the token
        ids are not sent (everything else is, in stream order behind the running burst)."""
        alloc = self.cache.alloc
        if not entries:
            raise StepError("a step needs at least one token")
        n_burst = 0 if burst_uniform is None else burst_uniform.shape[0]
        extra = max(n_burst - 1, 0)              # positions a burst adds beyond this step's
        seen = set()
        q_lens, kv_before, slots = [], [], []
        limit = self.model.max_positions
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if e.rid not in alloc:
                self.admit(e.rid)
            before = alloc.length(e.rid) + in_flight
            n = len(e.tokens)
            if limit is not None and before + n + extra > limit:
                raise StepError(f"request {e.rid!r}: {before + n + extra} tokens exceed the model's {limit} positions")
            q_lens.append(n)
            kv_before.append(before)
            slots.append(alloc.slot(e.rid))
        # all-or-nothing page reservation for the whole step (or burst)
        need = [0] * len(alloc.pools)
        for e, n, before in zip(entries, q_lens, kv_before):
            for g, k in enumerate(alloc.pages_needed(e.rid, before + n + extra)):
                need[g] += k
        for g, k in enumerate(need):
            if k > alloc.free_pages(g):
                raise OutOfPages(f"step needs {k} new pages in cache group {g}, "
                                 f"{alloc.free_pages(g)} of {alloc.pools[g].num_pages} are free")
        for e, n, before in zip(entries, q_lens, kv_before):
            alloc.reserve(e.rid, before + n + extra)

        T, S = sum(q_lens), len(entries)
        R = sum(len(e.want) for e in entries)
        if sampling is not None and len(sampling) != R:
            raise StepError(f"{len(sampling)} sampling rows for {R} wanted places")
        groups = self.cache.layout.groups
        decode_only = max(q_lens) == 1
        if n_burst and (not decode_only or R != S or sampling is None):
            raise StepError("a burst takes single tokens only, each with its logits wanted and sampled")
        if in_flight and not n_burst:
            raise StepError("only a burst can continue a burst")
        generation = self._staging.generation
        page = self.cache.page_size
        max_blocks = max(-(-(b + n + extra) // page) for b, n in zip(kv_before, q_lens))
        # widths in steps of 8 pages (32 for bursts, whose recordings are dearer): few distinct graphs
        grain = 32 if n_burst else 8
        max_blocks = max(8, -(-max_blocks // grain) * grain)
        n_sample = (4 * R if sampling is not None else 0) + (R + n_burst * R if n_burst else 0)
        total = 3 * T + S + (S + 1) + S + R + n_sample + len(groups) * S * max_blocks
        bi = self._staging.acquire(total)
        h = self._staging.host_np[bi]
        dev = self._staging.dev
        off = 0

        def take(n):
            nonlocal off
            sl = (off, n)
            off += n
            return h[sl[0]:sl[0] + n], sl

        ids_v, ids_s = take(T)
        pos_v, pos_s = take(T)
        seq_v, seq_s = take(T)
        slot_v, slot_s = take(S)
        qs_v, qs_s = take(S + 1)
        kvb_v, kvb_s = take(S)
        rows_v, rows_s = take(R)
        vocab = self.vocab_size
        if decode_only:
            ids_v[:] = [e.tokens[0] for e in entries]
            if int(ids_v.min()) < 0 or int(ids_v.max()) >= vocab:
                raise StepError(f"a token id is outside the vocabulary of {vocab}")
            pos_v[:] = kv_before
            seq_v[:] = np.arange(S, dtype=np.int32)
            qs_v[:] = np.arange(S + 1, dtype=np.int32)
            r0 = 0
            for s, e in enumerate(entries):
                for w in e.want:
                    if int(w) != 0:
                        raise StepError(f"request {e.rid!r}: wanted place {w} is outside its 1 token")
                    rows_v[r0] = s
                    r0 += 1
        else:
            t0, r0 = 0, 0
            for s, (e, n, before) in enumerate(zip(entries, q_lens, kv_before)):
                toks = np.asarray(e.tokens, dtype=np.int64)
                if toks.min() < 0 or toks.max() >= vocab:
                    raise StepError(f"request {e.rid!r}: a token id is outside the vocabulary of {vocab}")
                ids_v[t0:t0 + n] = toks
                pos_v[t0:t0 + n] = np.arange(before, before + n, dtype=np.int32)
                seq_v[t0:t0 + n] = s
                qs_v[s] = t0
                for w in e.want:
                    if not (0 <= int(w) < n):
                        raise StepError(f"request {e.rid!r}: wanted place {w} is outside its {n} tokens")
                    rows_v[r0] = t0 + int(w)
                    r0 += 1
                t0 += n
            qs_v[S] = T
        slot_v[:] = slots
        kvb_v[:] = kv_before
        sample_s = None
        if sampling is not None:
            sv, sample_s = take(4 * R)
            fv = sv.view(np.float32)
            fv[:R] = [row.temperature for row in sampling]
            sv[R:2 * R] = [row.top_k for row in sampling]
            fv[2 * R:3 * R] = [row.top_p for row in sampling]
            fv[3 * R:] = [row.uniform for row in sampling]
        step_s = None
        if n_burst:
            stv, step_s = take(R)
            stv[:] = 0
        table_slices = {}
        for g in groups:
            tv, ts = take(S * max_blocks)
            tv = tv.reshape(S, max_blocks)
            tv[:] = FREED
            for s, e in enumerate(entries):
                row = self._table_row(e.rid, g.index)
                m = min(row.shape[0], max_blocks)
                tv[s, :m] = row[:m]
            table_slices[g.index] = ts
        uni_s = None
        if n_burst:
            # last in the buffer: its length changes with the burst, nothing else may move with it
            uv, uni_s = take(n_burst * R)
            uv.view(np.float32)[:] = burst_uniform.reshape(-1)
        if in_flight and self._staging.generation != generation:
            raise StepError("the step buffer moved under a running burst")
        self._staging.send(bi, total, start=T if in_flight else 0)
        self.last_h2d_bytes = 4 * (total - (T if in_flight else 0))
        self.h2d_bytes_total += self.last_h2d_bytes

        def d(sl):
            return dev[sl[0]:sl[0] + sl[1]]

        ctx = StepContext(
            n_tokens=T, n_seqs=S,
            token_ids=d(ids_s), positions=d(pos_s), token_seq=d(seq_s), seq_slots=d(slot_s),
            q_start=d(qs_s), kv_before=d(kvb_s), logit_rows=d(rows_s),
            block_tables={g: d(sl).view(S, max_blocks) for g, sl in table_slices.items()},
            compute_dtype=self.dtype, workspace=self.workspace, caches=self.cache.device_caches,
            host_q_lens=q_lens, host_kv_before=kv_before, host_slots=slots,
            max_q_len=max(q_lens), max_kv_len=max(b + n for b, n in zip(kv_before, q_lens)) + extra,
        )
        sample_dev = d(sample_s) if sample_s is not None else None
        # Everything a launch's shape depends on.  The portions' own lengths and starts are device
        # data (q_start, kv_before, positions), so steps that agree on these counts share a graph:
        # decode steps always do, prompt steps do when the token budget is filled the same way.
        # A burst is recorded whole (all its steps in one graph), in two copies used in turn: a
        # graph that is launched again while it still runs makes the host wait for it.
        if n_burst:
            self._burst_flip ^= 1
        key = (T, S, R, max(q_lens), max_blocks, sampling is not None, n_burst,
               self._burst_flip if n_burst else 0, self._staging.generation)
        burst = (d(uni_s).view(torch.float32), d(step_s)) if n_burst else None
        return _Prepared(ctx, sample_dev, key, burst)

    # ---- running it ------------------------------------------------------------------------
    def _run(self, p: _Prepared) -> torch.Tensor:
        ctx = p.ctx
        logits = self.model.forward(ctx, status=self._status)
        R = ctx.logit_rows.numel()
        if p.sample is not None and R:
            f = p.sample.view(torch.float32)
            if p.burst is not None:
                uniform, row_step = p.burst
                ops.sample(logits, self._sampled[:R], temperature=f[:R], top_k=p.sample[R:2 * R],
                           top_p=f[2 * R:3 * R], uniform=uniform, status=self._status,
                           feedback=(ctx.token_ids, ctx.logit_rows, ctx.positions, self._burst_tokens, row_step))
            else:
                ops.sample(logits, self._sampled[:R], temperature=f[:R], top_k=p.sample[R:2 * R],
                           top_p=f[2 * R:3 * R], uniform=f[3 * R:4 * R], status=self._status)
        return logits

    def _graph_for(self, key: Tuple, record_at: int):
        """The valid recorded graph of `key`, or None; counts how often the key came by and says
        whether this is the time to record it."""
        hit = self._graphs.get(key)
        if hit is not None and hit[3] != self.workspace.version:
            # a workspace buffer has moved since this graph was recorded: its pointers are stale
            del self._graphs[key]
            self._seen.pop(key, None)
            hit = None
            self.stale_graphs += 1
        if hit is not None:
            return hit, False
        seen = self._seen.get(key, 0)
        self._seen[key] = seen + 1
        return None, seen >= record_at

    def _record(self, key: Tuple, p: _Prepared, times: int):
        before = ops.LAUNCHES
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(times):
                logits = self._run(p)
        n_launch = (ops.LAUNCHES - before) // times
        while len(self._graphs) >= MAX_GRAPHS:          # the oldest recording makes room
            del self._graphs[next(iter(self._graphs))]
            self._seen.clear()
        hit = (graph, logits, n_launch, self.workspace.version)
        self._graphs[key] = hit
        if times > 1:
            self.burst_graphs_recorded += 1
        return hit

    def _execute(self, p: _Prepared, times: int = 1) -> torch.Tensor:
        """Run the prepared step `times` times (more than once only for a burst, whose sampler
        moves the step's inputs on), through recorded graphs where there are any.

        Two kinds of recordings.  One step: recorded the second time its shape comes by, replayed
        `times` times for a burst.  A whole burst (all its steps in one graph, one launch): recorded
        once the same burst shape has come by three times, so that only workloads that stay in one
        shape pay for it; kept in two copies used in turn (the key carries the turn), because a
        graph launched again while it still runs makes the host wait for it, and the host has the
        next burst to prepare."""
        before = ops.LAUNCHES
        key = p.key
        if key is None or not self.use_cuda_graphs:
            logits = None
            for _ in range(times):
                logits = self._run(p)
            self.last_launches = (ops.LAUNCHES - before) // times
            return logits
        step_key = key
        if p.burst is not None:
            step_key = key[:6] + (1, 0) + key[8:]           # any burst length, either turn
            hit, record = self._graph_for(key, record_at=2)
            if hit is None and record:
                hit = self._record(key, p, times)
            if hit is not None:
                hit[0].replay()
                self.graph_replays += times
                self.last_launches = hit[2]
                return hit[1]
        hit, record = self._graph_for(step_key, record_at=1)
        if hit is None and record:
            hit = self._record(step_key, p, 1)
        if hit is not None:
            for _ in range(times):
                hit[0].replay()
            self.graph_replays += times
            self.last_launches = hit[2]
            return hit[1]
        logits = None
        for _ in range(times):
            logits = self._run(p)
        self.last_launches = (ops.LAUNCHES - before) // times
        return logits

    def step(self, entries: Sequence[StepEntry], sampling: Optional[Sequence[SampleRow]] = None) -> torch.Tensor:
        """Run one step; returns float32 logits [wanted, vocab] on the device.  The tensor is
        workspace memory: the next step overwrites it.  With `sampling` (one SampleRow per
        wanted place) the drawn tokens are in `self.sampled_tokens(n)` afterwards."""
        entries = [e for e in entries if len(e.tokens) > 0]
        p = self._prepare(entries, sampling)
        R = p.ctx.logit_rows.numel()
        if self._sampled.numel() < R:
            self._sampled = torch.zeros(R, dtype=torch.int32, device=self.device)
        logits = self._execute(p)
        for e, n, b in zip(entries, p.ctx.host_q_lens, p.ctx.host_kv_before):
            self.cache.alloc.commit(e.rid, b + n)
        self.steps_run += 1
        return logits

    def decode_burst(self, entries: Sequence[StepEntry], sampling: Sequence[SampleRow],
                     uniforms: np.ndarray) -> np.ndarray:
        """Run `n = uniforms.shape[0]` decode steps of the same requests back to back on the
        device.  Every entry brings one token and wants its logits; step j of request r is drawn
        with sampling[r] and the uniform number uniforms[j, r]; the token drawn in step j is the
        input of step j + 1.  Returns the drawn tokens, int32 [n, requests], on the host.

        Pages for all n steps are reserved before anything runs (OutOfPages otherwise, with
        nothing taken).  The requests' lengths are NOT advanced here: the caller commits as many
        of each request's steps as it keeps (`commit`), since a request may have hit a stop token
        part of the way through; what the later steps wrote for it lies beyond its length and is
        never read."""
        return self.burst_tokens(self.decode_burst_async(entries, sampling, uniforms))

    def decode_burst_async(self, entries: Sequence[StepEntry], sampling: Sequence[SampleRow],
                           uniforms: np.ndarray, in_flight: int = 0) -> "BurstHandle":
        """decode_burst without the wait: everything is queued on the stream, including the copy of
        the drawn tokens to pinned host memory, and a handle comes back for `burst_tokens`.
        With `in_flight` > 0 the burst continues one of the same requests, in the same order,
        that was queued before and is `in_flight` steps long (see _prepare): the host can queue
        the next burst before it has seen the tokens of the last, so its own work between two
        bursts (scheduling, packing, reading tokens) no longer leaves the device idle.  The
        entries' token ids are ignored then."""
        n = int(uniforms.shape[0])
        S = len(entries)
        if not (1 <= n <= MAX_BURST):
            raise StepError(f"a burst runs 1 to {MAX_BURST} steps, got {n}")
        if self._burst_tokens.numel() < n * S:
            raise StepError("more requests in a burst than the engine was built for")
        p = self._prepare(entries, sampling, burst_uniform=np.ascontiguousarray(uniforms, dtype=np.float32),
                          in_flight=in_flight)
        self._execute(p, times=n)
        host = self._burst_hosts[self._burst_turn]
        self._burst_turn ^= 1
        host[:n * S].copy_(self._burst_tokens[:n * S], non_blocking=True)
        self._copy_status(host, n * S)
        self.d2h_bytes_total += 4 * n * S + 8
        done = torch.cuda.Event()
        done.record()
        self.steps_run += n
        return BurstHandle(n, S, host, done)

    def burst_tokens(self, handle: "BurstHandle") -> np.ndarray:
        """Wait for a burst queued by decode_burst_async; its tokens, int32 [n, requests]."""
        handle.done.synchronize()
        self._raise_on_status(handle.host, handle.n * handle.S)
        return handle.host[:handle.n * handle.S].numpy().reshape(handle.n, handle.S).copy()

    def commit(self, rid: Hashable, new_len: int) -> None:
        """Advance a request's length after a burst (see decode_burst)."""
        self.cache.alloc.commit(rid, new_len)

    def _copy_status(self, host: torch.Tensor, at: int) -> None:
        """Queue copies of the two status words (bad input, kernel faults) to host[at], host[at + 1],
        behind whatever the stream holds: they travel with the drawn tokens, at no extra wait."""
        host[at:at + 1].copy_(self._status, non_blocking=True)
        host[at + 1:at + 2].copy_(ops.kernel_status(self.device), non_blocking=True)

    def _raise_on_status(self, host: torch.Tensor, at: int) -> None:
        bad_input, fault = int(host[at]), int(host[at + 1])
        if bad_input or fault:
            self.check_status()          # clears the words and raises with their meaning

    def read_sampled(self, n: int) -> List[int]:
        """The tokens drawn by the last step with `sampling`, on the host.  The step's status words
        come back in the same wait; a non-zero one raises (the tokens are not valid then)."""
        if self._token_host.numel() < n + 2:
            self._token_host = torch.zeros(n + 2, dtype=torch.int32, pin_memory=True)
        host = self._token_host
        host[:n].copy_(self._sampled[:n], non_blocking=True)
        self._copy_status(host, n)
        self.d2h_bytes_total += 4 * n + 8
        torch.cuda.current_stream().synchronize()
        self._raise_on_status(host, n)
        return host[:n].tolist()

    def sampled_tokens(self, n: int) -> torch.Tensor:
        """The tokens drawn by the last step with `sampling` (int32 [n] on the device)."""
        return self._sampled[:n]

    def check_status(self) -> None:
        """Raise if a kernel reported bad input or an expired wait since the last check."""
        code = int(self._status.item())
        if code:
            self._status.zero_()
            raise StepError(f"a kernel reported bad input (status {code}: bit0 token id or NaN logits, bit1 position)")
        ops.check_kernel_status(self.device)
