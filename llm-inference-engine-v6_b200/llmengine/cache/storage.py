"""Device side of the cache: page tensors per layer run, grouped by what the runs must keep.

The cache manager (host, C++) hands out page ids and slot ids; this module decides the groups and
allocates what the ids index. Runs whose mixers keep all keys form one group, runs with a window
of W form another (one per distinct W); each group has its own pool of pages and its own block
table per request. Every page tensor has one page more than the pool: the null page, which padded
batch rows write to. State tensors likewise have one slot more than the pool.

Layout of one run's keys (and values): [page, kv_head, slot_in_page, head_dim]: a page of one
kv head is contiguous, so one TMA box or one coalesced burst fetches it. The reference keeps one
float32 pool for all layers with layout [K l0..][V l0..] per block (src/paged_kv.cpp:22-66).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVNeed, LayerCache, StateNeed


@dataclass
class CacheGroup:
    window: int
    num_pages: int


def plan_groups(run_needs: Sequence[Sequence[object]]) -> Tuple[List[int], List[Optional[int]]]:
    """run_needs[r] = cache needs of run r (empty for a run that borrows a cache or keeps none).
    -> (windows of the groups, group index of every run or None)."""
    windows: List[int] = []
    run_group: List[Optional[int]] = []
    for needs in run_needs:
        kv = [n for n in needs if isinstance(n, KVNeed)]
        if len(kv) > 1:
            raise ValueError("a layer may keep at most one set of keys and values")
        if not kv:
            run_group.append(None)
            continue
        w = kv[0].window
        if w not in windows:
            windows.append(w)
        run_group.append(windows.index(w))
    if not windows:
        windows.append(0)  # a model without attention still gets a (tiny, unused) pool: tables stay uniform
    return windows, run_group


def bytes_per_token(run_needs: Sequence[Sequence[object]], dtype: torch.dtype) -> int:
    el = torch.empty((), dtype=dtype).element_size()
    total = 0
    for needs in run_needs:
        for n in needs:
            if isinstance(n, KVNeed):
                total += 2 * n.num_kv_heads * n.head_dim * el
    return total


def allocate_run_caches(run_needs: Sequence[Sequence[object]], run_group: Sequence[Optional[int]],
                        group_pages: Sequence[int], windows: Sequence[int], page_size: int, num_slots: int,
                        dtype: torch.dtype, device: torch.device) -> List[LayerCache]:
    caches: List[LayerCache] = []
    for needs, g in zip(run_needs, run_group):
        c = LayerCache()
        for n in needs:
            if isinstance(n, KVNeed):
                shape = (group_pages[g] + 1, n.num_kv_heads, page_size, n.head_dim)
                c.group, c.window = g, windows[g]
                c.k = torch.zeros(shape, dtype=dtype, device=device)
                c.v = torch.zeros(shape, dtype=dtype, device=device)
            elif isinstance(n, StateNeed):
                c.states[n.name] = torch.zeros((num_slots + 1,) + tuple(n.shape), dtype=n.dtype, device=device)
            else:
                raise TypeError(f"unknown cache need {n!r}")
        caches.append(c)
    return caches
