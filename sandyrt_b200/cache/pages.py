"""The cache manager's host side: page pools, per-request block lists, state slots.

The bookkeeping is the host library's (core/cache.cpp: PagePool, CacheLayout, BlockAllocator); the
classes here are its Python face, so that every decision about pages can be driven and tested from
Python on a machine without a GPU.

What the reference does (one request at a time): a pool of fixed-size pages with a LIFO free list,
optional page cap, double-free detection (src/core/Allocator.cpp:60-122,
src/device/cuda/CudaPagedTensor.cpp:232-267); growth by ceil(new_len / page_size) pages (:95-137,
:555-576); everything returned when the request's session ends (:528-553,
src/server/Session.cpp:552-563); one list of cache groups per model (`CacheGroupConfig`,
src/server/Session.h:36-41, src/server/Model.cpp:106-111).

What is different here: the lowest free page goes out first (so that a prompt's pages tend to be a
run); many requests live at once and share the pools; a request has one block list per *group* (all
layers of a group use the same page ids), not one page table per tensor; pages of a group whose
layers only look back `window` positions are given back as soon as the window has passed them; and
every request also holds one *state slot*, a row index into per-request state of fixed size.

Request ids may be any hashable value here; the library knows them by integers.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .. import core
from ..errors import CacheError, NoFreeSlot, OutOfPages  # noqa: F401  (re-exported)
from ..parts.base import PagedKVSpec, StateSpec, cache_spec_json

FREED = -1   # entry of a block list whose page has been given back (window has passed it)


class RequestIds:
    """Hashable request ids <-> the integers the library knows requests by."""

    def __init__(self):
        self._to_int: Dict[Hashable, int] = {}
        self._to_rid: Dict[int, Hashable] = {}
        self._next = 1

    def of(self, rid: Hashable) -> int:
        i = self._to_int.get(rid)
        if i is None:
            i = self._next
            self._next += 1
            self._to_int[rid] = i
            self._to_rid[i] = rid
        return i

    def rid(self, i: int) -> Hashable:
        return self._to_rid[i]

    def known(self, rid: Hashable) -> bool:
        return rid in self._to_int

    def forget(self, rid: Hashable) -> None:
        i = self._to_int.pop(rid, None)
        if i is not None:
            self._to_rid.pop(i, None)


class PagePool:
    """Page ids 0..num_pages-1; the free page with the lowest id is handed out first (the
    reference's pool is a LIFO list).  A fresh pool hands out 0, 1, 2, ..., and whenever the low end
    of the pool is free again a request's pages follow one another in the cache: the prompt
    attention kernel fetches such runs with one copy per tile.  With few pages (the tests) a page
    just freed is still handed out again at once."""

    def __init__(self, num_pages: int):
        self._h = core.Handle("pool", core.call("global", None, "new_pool", num_pages=num_pages)["handle"])
        self.num_pages = num_pages

    free_pages = property(lambda self: self._h.call("info")["free_pages"])
    used_pages = property(lambda self: self._h.call("info")["used_pages"])
    high_water = property(lambda self: self._h.call("info")["high_water"])

    def allocate(self, n: int) -> List[int]:
        return self._h.call("allocate", n=n)

    def release(self, pages: Sequence[int]) -> None:
        self._h.call("release", pages=[int(p) for p in pages])


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
    specs: Sequence[object] = ()

    @classmethod
    def from_specs(cls, specs: Sequence[object], page_size: int) -> "CacheLayout":
        for ci, s in enumerate(specs):
            if s is not None and not isinstance(s, (PagedKVSpec, StateSpec)):
                raise CacheError(f"cache entry {ci}: unknown cache spec {s!r}")
        probe = core.Handle("allocator", core.call("global", None, "new_allocator", specs=[cache_spec_json(s) for s in specs],
                                                   pages=1, page_size=page_size, max_requests=1)["handle"])
        return cls._from_json(probe.call("layout"), specs)

    @classmethod
    def _from_json(cls, j, specs=()) -> "CacheLayout":
        groups = [CacheGroup(g["index"], PagedKVSpec(g["n_kv_heads"], g["head_dim"], g["window"] or None), list(g["caches"]))
                  for g in j["groups"]]
        states = {}
        for ci in j["state_caches"]:
            states[ci] = specs[ci] if ci < len(specs) else StateSpec(())
        return cls(j["page_size"], groups, {int(k): tuple(v) for k, v in j["group_of_cache"].items()}, states, tuple(specs))


class _PoolView:
    def __init__(self, alloc: "BlockAllocator", group: int):
        self._alloc, self._group = alloc, group

    def _info(self):
        return self._alloc._h.call("pools")[self._group]

    num_pages = property(lambda self: self._info()["num_pages"])
    free_pages = property(lambda self: self._info()["free_pages"])
    used_pages = property(lambda self: self._info()["used_pages"])
    high_water = property(lambda self: self._info()["high_water"])


class BlockAllocator:
    """Pages and slots of all live requests.

      admit(rid)              take a state slot; the request holds no pages yet
      reserve(rid, new_len)   make room for positions < new_len in every group (all or nothing)
      commit(rid, new_len)    the step ran: the request now holds new_len tokens; pages a
                              window has passed are given back
      release(rid)            the request ended: everything it holds is given back
    """

    def __init__(self, layout: Optional[CacheLayout] = None, pages_per_group: Sequence[int] = (), max_requests: int = 4, *,
                 _handle: Optional[core.Handle] = None, _ids: Optional[RequestIds] = None):
        if _handle is None:
            if len(pages_per_group) != len(layout.groups):
                raise CacheError("one page count per cache group is needed")
            _handle = core.Handle("allocator", core.call(
                "global", None, "new_allocator", specs=[cache_spec_json(s) for s in layout.specs],
                pages=list(pages_per_group), page_size=layout.page_size, max_requests=max_requests)["handle"])
        self._h = _handle
        self.ids = _ids or RequestIds()
        info = self._h.call("info")
        self.page_size, self.max_requests = info["page_size"], info["max_requests"]
        self.layout = layout if layout is not None else CacheLayout._from_json(self._h.call("layout"))
        self.pools = [_PoolView(self, g) for g in range(info["n_groups"])]

    def _call(self, method: str, rid: Hashable, **kw):
        if not self.ids.known(rid) and method != "admit":
            if method == "contains":
                return False
            raise CacheError(f"request {rid!r} is not live")
        try:
            return self._h.call(method, rid=self.ids.of(rid), **kw)
        except CacheError as e:
            raise CacheError(str(e).replace(f"request {self.ids.of(rid)} ", f"request {rid!r} ")) from None

    # ---- queries ---------------------------------------------------------------------
    def __contains__(self, rid) -> bool:
        return self.ids.known(rid) and self._h.call("contains", rid=self.ids.of(rid))

    def live(self) -> List[Hashable]:
        return [self.ids.rid(i) for i in self._h.call("live")]

    def slot(self, rid) -> int:
        return self._call("slot", rid)

    def length(self, rid) -> int:
        return self._call("length", rid)

    def block_version(self, rid) -> int:
        return self._call("block_version", rid)

    def block_list(self, rid, group: int) -> List[int]:
        return self._call("block_list", rid, group=group)

    def free_slots(self) -> int:
        return self._h.call("free_slots")

    def free_pages(self, group: int = 0) -> int:
        return self._h.call("free_pages", group=group)

    def pages_needed(self, rid, new_len: int) -> List[int]:
        return self._call("pages_needed", rid, new_len=new_len)

    def can_reserve(self, rid, new_len: int) -> bool:
        return self._call("can_reserve", rid, new_len=new_len)

    # ---- transitions -----------------------------------------------------------------
    def admit(self, rid) -> int:
        return self._call("admit", rid)

    def reserve(self, rid, new_len: int) -> None:
        self._call("reserve", rid, new_len=new_len)

    def commit(self, rid, new_len: int) -> None:
        self._call("commit", rid, new_len=new_len)

    def release(self, rid) -> None:
        self._call("release", rid)

    def check(self) -> None:
        """No page lost, held twice or free while held; no slot lost or shared."""
        self._h.call("check")
