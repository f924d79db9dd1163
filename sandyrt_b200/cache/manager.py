"""Device side of the cache: the page arenas and per-request states, beside the host-side
BlockAllocator that decides who holds which page.

One arena per cache group: [caches in group][num_pages][K|V][Hkv][page_size][D] in the
compute dtype, allocated once.  (The reference allocates every page separately on demand
with cudaMallocAsync and keeps a table of page *pointers* per tensor,
src/device/cuda/CudaPagedTensor.cpp:232-267,345-447; here a page is an index into one
arena and a request has one int32 block list per group, shared by all layers of the group.)

Fixed-size per-request state: one tensor [max_requests, *shape] per cache entry whose mixer
declares a StateSpec; row `slot` belongs to the request holding that slot and is zeroed
when the request is admitted.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..parts.base import PagedKVSpec, StateSpec
from .pages import BlockAllocator, CacheLayout, FREED


class DeviceCaches:
    def __init__(self, layout: CacheLayout, pages_per_group: Sequence[int], max_requests: int,
                 device, dtype: torch.dtype):
        self.layout = layout
        self.arenas: List[torch.Tensor] = []
        for g, n_pages in zip(layout.groups, pages_per_group):
            s = g.spec
            self.arenas.append(torch.zeros(
                (len(g.caches), n_pages, 2, s.n_kv_heads, layout.page_size, s.head_dim),
                dtype=dtype, device=device))
        self.states: Dict[int, torch.Tensor] = {
            ci: torch.zeros((max_requests,) + tuple(spec.shape), dtype=spec.dtype, device=device)
            for ci, spec in layout.state_of_cache.items()}

    def kv(self, cache: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
        """(K view, V view, group) of a cache entry; views are [num_pages, Hkv, page_size, D]."""
        g, i = self.layout.group_of_cache[cache]
        arena = self.arenas[g]
        return arena[i, :, 0], arena[i, :, 1], g

    def state(self, cache: int) -> torch.Tensor:
        return self.states[cache]

    def zero_slot(self, slot: int) -> None:
        for t in self.states.values():
            t[slot].zero_()

    def poison(self) -> None:
        """Fill every page with NaN (tests: a read of a slot nobody wrote then shows)."""
        for a in self.arenas:
            a.fill_(float("nan"))

    def bytes(self) -> int:
        return sum(a.numel() * a.element_size() for a in self.arenas) + \
            sum(t.numel() * t.element_size() for t in self.states.values())


class CacheManager:
    """BlockAllocator + DeviceCaches for one model on one device."""

    def __init__(self, cache_specs: Sequence[object], *, page_size: int, max_tokens: int,
                 max_requests: int, device, dtype: torch.dtype):
        self.layout = CacheLayout.from_specs(cache_specs, page_size)
        n_pages = max(1, -(-max_tokens // page_size))
        self.pages_per_group = [n_pages for _ in self.layout.groups]
        self.alloc = BlockAllocator(self.layout, self.pages_per_group, max_requests)
        self.device_caches = DeviceCaches(self.layout, self.pages_per_group, max_requests, device, dtype)
        self.page_size = page_size
        self.max_requests = max_requests

    def admit(self, rid: Hashable) -> int:
        slot = self.alloc.admit(rid)
        self.device_caches.zero_slot(slot)
        return slot

    def release(self, rid: Hashable) -> None:
        self.alloc.release(rid)

    def kv_bytes_per_token(self) -> int:
        total = 0
        for g, a in zip(self.layout.groups, self.device_caches.arenas):
            total += len(g.caches) * 2 * g.spec.n_kv_heads * g.spec.head_dim * a.element_size()
        return total
