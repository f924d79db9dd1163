"""The step function: one batch of (request, its next tokens) through the model.

`Engine.step(entries)` takes, for each request of the step, the tokens that follow what
the request already has in the cache (a portion of a prompt of any length, or one decoded
token) and the places among them whose logits are wanted.  It runs exactly those tokens as
one batch, reading everything earlier from the cache, appends their keys and values to the
cache, and returns float32 logits [wanted, vocab] in the order of the entries and of their
wanted places.

The reference's counterpart, Engine::runValues on one of two compiled graphs (decode with
input_id [1,1], prefill with input_id [1,n]; src/engine/Engine.h:100-104,
src/server/Model.cpp:216-255, inputs built in src/server/Session.cpp:167-206), serves one
request per call and returns logits for every row.  Here there is one code path for every
mix of requests, and rows nobody asked for are never computed past the last layer.

All the step's index arrays (token ids, positions, request of each token, block tables,
wanted rows) are packed on the host into one pinned buffer and reach the device with one
copy.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import FREED, OutOfPages
from ..models.model import Model
from ..parts.base import StepContext, Workspace


@dataclasses.dataclass
class StepEntry:
    """One request's share of a step."""
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()        # indices into `tokens` whose logits are returned


class StepError(Exception):
    pass


class _Staging:
    """A ring of pinned host buffers and one device buffer for the step's index arrays."""

    def __init__(self, device, depth: int = 4):
        self.device = device
        self.depth = depth
        self.capacity = 0
        self.host: List[torch.Tensor] = []
        self.events: List[Optional[torch.cuda.Event]] = []
        self.dev: Optional[torch.Tensor] = None
        self.turn = 0

    def acquire(self, n: int):
        if n > self.capacity:
            self.capacity = max(1024, 1 << (n - 1).bit_length())
            self.host = [torch.empty(self.capacity, dtype=torch.int32, pin_memory=True) for _ in range(self.depth)]
            self.events = [None] * self.depth
            self.dev = torch.empty(self.capacity, dtype=torch.int32, device=self.device)
        i = self.turn
        self.turn = (self.turn + 1) % self.depth
        if self.events[i] is not None:
            self.events[i].synchronize()      # the copy that last used this buffer is done
        return i, self.host[i], self.dev

    def sent(self, i: int) -> None:
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class Engine:
    """A bound model, its cache and the step function over them."""

    def __init__(self, model: Model, *, max_tokens: int, page_size: int = 16, max_requests: int = 64,
                 use_cuda_graphs: bool = False):
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
        self._staging = _Staging(self.device)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self.last_h2d_bytes = 0

    # ---- request lifetime ------------------------------------------------------------
    def admit(self, rid: Hashable) -> int:
        return self.cache.admit(rid)

    def release(self, rid: Hashable) -> None:
        self.cache.release(rid)

    def length(self, rid: Hashable) -> int:
        return self.cache.alloc.length(rid)

    # ---- the step --------------------------------------------------------------------
    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Reserve pages, pack the step's index arrays and copy them to the device."""
        alloc = self.cache.alloc
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            raise StepError("a step needs at least one token")
        seen = set()
        q_lens, kv_before, slots = [], [], []
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if e.rid not in alloc:
                self.admit(e.rid)
            before = alloc.length(e.rid)
            n = len(e.tokens)
            limit = self.model.max_positions
            if limit is not None and before + n > limit:
                raise StepError(f"request {e.rid!r}: {before + n} tokens exceed the model's {limit} positions")
            for t in e.tokens:
                if not (0 <= int(t) < self.vocab_size):
                    raise StepError(f"request {e.rid!r}: token id {t} is outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.rid!r}: wanted place {w} is outside its {n} tokens")
            q_lens.append(n)
            kv_before.append(before)
            slots.append(alloc.slot(e.rid))
        # all-or-nothing page reservation for the whole step
        need = [0] * len(alloc.pools)
        for e, n, before in zip(entries, q_lens, kv_before):
            for g, k in enumerate(alloc.pages_needed(e.rid, before + n)):
                need[g] += k
        for g, k in enumerate(need):
            if k > alloc.free_pages(g):
                raise OutOfPages(f"step needs {k} new pages in cache group {g}, "
                                 f"{alloc.free_pages(g)} of {alloc.pools[g].num_pages} are free")
        for e, n, before in zip(entries, q_lens, kv_before):
            alloc.reserve(e.rid, before + n)

        T, S = sum(q_lens), len(entries)
        groups = self.cache.layout.groups
        max_blocks = max(1, max(-(-(b + n) // self.cache.page_size) for b, n in zip(kv_before, q_lens)))
        R = sum(len(e.want) for e in entries)
        total = 3 * T + S + (S + 1) + S + R + len(groups) * S * max_blocks
        bi, host, dev = self._staging.acquire(total)
        h = host.numpy()
        off = 0

        def take(n):
            nonlocal off
            view = h[off:off + n]
            sl = (off, n)
            off += n
            return view, sl

        ids_v, ids_s = take(T)
        pos_v, pos_s = take(T)
        seq_v, seq_s = take(T)
        slot_v, slot_s = take(S)
        qs_v, qs_s = take(S + 1)
        kvb_v, kvb_s = take(S)
        rows_v, rows_s = take(R)
        t0, r0 = 0, 0
        for s, (e, n, before) in enumerate(zip(entries, q_lens, kv_before)):
            ids_v[t0:t0 + n] = np.asarray(e.tokens, dtype=np.int32)
            pos_v[t0:t0 + n] = np.arange(before, before + n, dtype=np.int32)
            seq_v[t0:t0 + n] = s
            qs_v[s] = t0
            for w in e.want:
                rows_v[r0] = t0 + int(w)
                r0 += 1
            t0 += n
        qs_v[S] = T
        slot_v[:] = slots
        kvb_v[:] = kv_before
        table_slices = {}
        for g in groups:
            tv, ts = take(S * max_blocks)
            tv = tv.reshape(S, max_blocks)
            tv[:] = FREED
            for s, e in enumerate(entries):
                bl = alloc.block_list(e.rid, g.index)
                m = min(len(bl), max_blocks)
                tv[s, :m] = bl[:m]
            table_slices[g.index] = ts
        dev[:total].copy_(host[:total], non_blocking=True)
        self.last_h2d_bytes = 4 * total
        self._staging.sent(bi)

        def d(sl):
            return dev[sl[0]:sl[0] + sl[1]]

        return StepContext(
            n_tokens=T, n_seqs=S,
            token_ids=d(ids_s), positions=d(pos_s), token_seq=d(seq_s), seq_slots=d(slot_s),
            q_start=d(qs_s), kv_before=d(kvb_s), logit_rows=d(rows_s),
            block_tables={g: d(sl).view(S, max_blocks) for g, sl in table_slices.items()},
            compute_dtype=self.dtype, workspace=self.workspace, caches=self.cache.device_caches,
            host_q_lens=q_lens, host_kv_before=kv_before, host_slots=slots,
            max_q_len=max(q_lens), max_kv_len=max(b + n for b, n in zip(kv_before, q_lens)),
        )

    def step(self, entries: Sequence[StepEntry], reserved: bool = False) -> torch.Tensor:
        """Run one step; returns float32 logits [wanted, vocab] on the device.  The tensor
        is workspace memory: it is overwritten by the next step."""
        entries = [e for e in entries if len(e.tokens) > 0]
        ctx = self.build_context(entries)
        logits = self.model.forward(ctx, status=self._status)
        for e, n, before in zip(entries, ctx.host_q_lens, ctx.host_kv_before):
            self.cache.alloc.commit(e.rid, before + n)
        self.steps_run += 1
        return logits

    def check_status(self) -> None:
        """Raise if a kernel reported a bad token id or position since the last check."""
        code = int(self._status.item())
        if code:
            self._status.zero_()
            raise StepError(f"a kernel reported bad input (status {code}: bit0 token id, bit1 position)")
