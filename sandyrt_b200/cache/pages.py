"""Host-side bookkeeping of the cache: page pools, per-request block lists, state slots.

Nothing in this file touches a device, so every decision about pages can be tested on a
machine without a GPU.

What the reference does (one request at a time): a pool of fixed-size pages with a LIFO
free list, optional page cap, double-free detection (src/core/Allocator.cpp:60-122,
src/device/cuda/CudaPagedTensor.cpp:232-267); growth by ceil(new_len / page_size) pages
(:95-137, :555-576); everything returned when the request's session ends (:528-553,
src/server/Session.cpp:552-563); one list of cache groups per model
(`CacheGroupConfig`, src/server/Session.h:36-41, src/server/Model.cpp:106-111).

What is different here: the lowest free page goes out first (so that a prompt's pages tend to
be a run); many requests live at once and share the pools; a request has one
block list per *group* (all layers of a group use the same page ids), not one page table
per tensor; pages of a group whose layers only look back `window` positions are given back
as soon as the window has passed them; and every request also holds one *state slot*, a
row index into per-request state of fixed size.
"""
from __future__ import annotations

import dataclasses
import heapq
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from ..parts.base import PagedKVSpec, StateSpec

FREED = -1   # entry of a block list whose page has been given back (window has passed it)


class OutOfPages(Exception):
    """A group's pool cannot supply the pages a reservation needs.  Nothing was taken."""


class NoFreeSlot(Exception):
    """Every state slot is held by a live request."""


class CacheError(Exception):
    """A misuse of the cache: unknown request, page freed twice, shrinking a request..."""


class PagePool:
    """Page ids 0..num_pages-1; the free page with the lowest id is handed out first (the
    reference's pool is a LIFO list).  A fresh pool hands out 0, 1, 2, ..., and whenever the low
    end of the pool is free again a request's pages follow one another in the cache: the
    prompt attention kernel fetches such runs with one copy per tile.  With few pages (the
    tests) a page just freed is still handed out again at once."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages))      # a heap (an ascending list is one)
        self._held = [False] * num_pages
        self.high_water = 0

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} of {self.num_pages} free")
        pages = [heapq.heappop(self._free) for _ in range(n)]
        for p in pages:
            self._held[p] = True
        self.high_water = max(self.high_water, self.used_pages)
        return pages

    def release(self, pages: Sequence[int]) -> None:
        pages = list(pages)
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise CacheError(f"page {p} does not belong to this pool")
            if not self._held[p]:
                raise CacheError(f"page {p} freed twice")
            self._held[p] = False
        for p in pages:
            heapq.heappush(self._free, p)


@dataclasses.dataclass
class CacheGroup:
    """Cache entries with the same needs; they share page ids and one pool."""
    index: int
    spec: PagedKVSpec
    caches: List[int]            # cache entries (of the model's run order) in this group


@dataclasses.dataclass
class CacheLayout:
    """How a model's cache entries fall into paged groups and fixed-size states."""
    page_size: int
    groups: List[CacheGroup]
    group_of_cache: Dict[int, Tuple[int, int]]     # cache entry -> (group, index inside group)
    state_of_cache: Dict[int, StateSpec]           # cache entry -> fixed-size state

    @classmethod
    def from_specs(cls, specs: Sequence[object], page_size: int) -> "CacheLayout":
        if page_size <= 0 or page_size & (page_size - 1):
            # the reference enforces a power of two as well (src/ir/MidIRMaterializer.cpp:48-49)
            raise CacheError(f"page size must be a power of two, got {page_size}")
        groups: List[CacheGroup] = []
        group_of_cache: Dict[int, Tuple[int, int]] = {}
        state_of_cache: Dict[int, StateSpec] = {}
        for ci, spec in enumerate(specs):
            if spec is None:
                continue
            if isinstance(spec, StateSpec):
                state_of_cache[ci] = spec
                continue
            if not isinstance(spec, PagedKVSpec):
                raise CacheError(f"cache entry {ci}: unknown cache spec {spec!r}")
            for g in groups:
                if g.spec == spec:
                    group_of_cache[ci] = (g.index, len(g.caches))
                    g.caches.append(ci)
                    break
            else:
                g = CacheGroup(len(groups), spec, [ci])
                groups.append(g)
                group_of_cache[ci] = (g.index, 0)
        return cls(page_size, groups, group_of_cache, state_of_cache)


@dataclasses.dataclass
class _Request:
    slot: int
    length: int                       # tokens whose keys/values are in the cache
    blocks: List[List[int]]           # per group: page id per block index, FREED where given back
    version: int = 0                  # changes whenever a block list changes (never reused)


class BlockAllocator:
    """Pages and slots of all live requests.

      admit(rid)              take a state slot; the request holds no pages yet
      reserve(rid, new_len)   make room for positions < new_len in every group (all or nothing)
      commit(rid, new_len)    the step ran: the request now holds new_len tokens; pages a
                              window has passed are given back
      release(rid)            the request ended: everything it holds is given back
    """

    def __init__(self, layout: CacheLayout, pages_per_group: Sequence[int], max_requests: int):
        if len(pages_per_group) != len(layout.groups):
            raise CacheError("one page count per cache group is needed")
        self.layout = layout
        self.page_size = layout.page_size
        self.pools = [PagePool(n) for n in pages_per_group]
        self.max_requests = max_requests
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}
        self._stamp = 0

    # ---- queries ---------------------------------------------------------------------
    def __contains__(self, rid) -> bool:
        return rid in self._requests

    def live(self) -> List[Hashable]:
        return list(self._requests)

    def _get(self, rid) -> _Request:
        try:
            return self._requests[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def slot(self, rid) -> int:
        return self._get(rid).slot

    def length(self, rid) -> int:
        return self._get(rid).length

    def block_version(self, rid) -> int:
        """A number that changes whenever any of the request's block lists changes; a request
        that is released and admitted again under the same id gets a new one."""
        return self._get(rid).version

    def block_list(self, rid, group: int) -> List[int]:
        return self._get(rid).blocks[group]

    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self, group: int = 0) -> int:
        return self.pools[group].free_pages

    def _first_needed_block(self, group: int, length: int) -> int:
        """Blocks below this index hold only positions no later query of a request of
        `length` tokens will read."""
        window = self.layout.groups[group].spec.window
        if not window:
            return 0
        first_pos = max(0, length - window + 1)   # oldest key the next query (position `length`) reads
        return first_pos // self.page_size

    def pages_needed(self, rid, new_len: int) -> List[int]:
        """Pages each group would have to supply for reserve(rid, new_len)."""
        r = self._get(rid)
        want_blocks = -(-new_len // self.page_size)
        return [max(0, want_blocks - len(bl)) for bl in r.blocks]

    def pages_for_new_request(self, n_tokens: int) -> List[int]:
        return [-(-n_tokens // self.page_size)] * len(self.pools)

    def can_reserve(self, rid, new_len: int) -> bool:
        return all(n <= p.free_pages for n, p in zip(self.pages_needed(rid, new_len), self.pools))

    # ---- transitions -----------------------------------------------------------------
    def admit(self, rid) -> int:
        if rid in self._requests:
            raise CacheError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.max_requests} state slots are in use")
        slot = self._free_slots.pop()
        self._stamp += 1
        self._requests[rid] = _Request(slot, 0, [[] for _ in self.pools], self._stamp)
        return slot

    def reserve(self, rid, new_len: int) -> None:
        r = self._get(rid)
        if new_len < r.length:
            raise CacheError(f"request {rid!r} holds {r.length} tokens, cannot reserve for {new_len}")
        need = self.pages_needed(rid, new_len)
        for g, (n, pool) in enumerate(zip(need, self.pools)):
            if n > pool.free_pages:
                raise OutOfPages(f"group {g}: request {rid!r} needs {n} more pages for {new_len} tokens, "
                                 f"{pool.free_pages} of {pool.num_pages} free")
        for bl, n, pool in zip(r.blocks, need, self.pools):
            if n:
                bl.extend(pool.allocate(n))
                self._stamp += 1
                r.version = self._stamp

    def commit(self, rid, new_len: int) -> None:
        r = self._get(rid)
        if new_len < r.length:
            raise CacheError(f"request {rid!r} cannot shrink from {r.length} to {new_len}")
        cap = min((len(bl) for bl in r.blocks), default=None)
        if cap is not None and new_len > cap * self.page_size:
            raise CacheError(f"request {rid!r}: {new_len} tokens were not reserved")
        r.length = new_len
        for g, bl in enumerate(r.blocks):
            first = min(self._first_needed_block(g, new_len), len(bl))
            gone = [p for p in bl[:first] if p != FREED]
            if gone:
                self.pools[g].release(gone)
                for i in range(first):
                    bl[i] = FREED
                self._stamp += 1
                r.version = self._stamp

    def release(self, rid) -> None:
        r = self._get(rid)
        for bl, pool in zip(r.blocks, self.pools):
            pool.release([p for p in bl if p != FREED])
        self._free_slots.append(r.slot)
        del self._requests[rid]

    # ---- self-check (tests call this after every operation) ---------------------------
    def check(self) -> None:
        """No page lost, held twice or free while held; no slot lost or shared."""
        for g, pool in enumerate(self.pools):
            held = [p for r in self._requests.values() for p in r.blocks[g] if p != FREED]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a page is held twice")
            free = pool._free
            if len(free) != len(set(free)):
                raise CacheError(f"group {g}: a page is on the free list twice")
            if set(held) & set(free):
                raise CacheError(f"group {g}: a held page is on the free list")
            if len(held) + len(free) != pool.num_pages:
                raise CacheError(f"group {g}: {pool.num_pages - len(held) - len(free)} pages lost")
        slots = [r.slot for r in self._requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots) \
                or len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("state slots are inconsistent")
