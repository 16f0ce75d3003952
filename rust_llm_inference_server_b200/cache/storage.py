"""Device storage behind the cache manager: pages of keys and values per group of layers with
the same needs, and slots of fixed-size per-request state.

Role of `PagedKvCache` (crates/model/src/paged.rs:23-152): there every layer has a K and a V
tensor (slot, kv head, d) and a page id addresses the same rows in all of them.  Here the cache
slots of the model's run order are sorted into groups by what they keep (head geometry, all
tokens or a window); a group has one pool of pages, [slot in group, K|V, page, kv head, position
in page, d], so one (page, head) tile is contiguous, and one block table per request.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import KVCacheSpec, LayerCache


@dataclass
class CacheGroup:
    spec: KVCacheSpec
    slots: list            # cache slot ids of the run order that live in this group
    page_size: int
    num_pages: int = 0

    @property
    def window(self) -> int:
        return int(self.spec.window) if self.spec.window else 0

    def bytes_per_page(self, elem_size: int) -> int:
        return len(self.slots) * 2 * self.spec.n_kv_heads * self.page_size * self.spec.head_dim * elem_size


def plan_groups(slot_specs, page_size: int) -> list[CacheGroup]:
    """Sorts cache slots into groups of identical needs, in order of first appearance."""
    groups: list[CacheGroup] = []
    for slot, spec in enumerate(slot_specs):
        if spec is None:
            continue
        for g in groups:
            if g.spec == spec:
                g.slots.append(slot)
                break
        else:
            groups.append(CacheGroup(spec, [slot], page_size))
    return groups


def size_groups(groups: list[CacheGroup], kv_cache_bytes: int, elem_size: int,
                max_num_seqs: int | None = None, max_batched_tokens: int | None = None) -> None:
    """Pages for every group out of `kv_cache_bytes`: the same number each
    (crates/model/src/paged.rs:109-116 for the single-group case), except that a window group is
    not given more than its requests can ever hold at once (a window plus one portion of a prompt,
    and the page either end may straddle, per seat); what that saves goes to the groups that keep
    every token."""
    per_page = sum(g.bytes_per_page(elem_size) for g in groups)
    n = kv_cache_bytes // per_page if per_page else 0
    for g in groups:
        g.num_pages = int(n)
    if not max_num_seqs or not max_batched_tokens:
        return
    saved = 0
    for g in groups:
        if g.window:
            most = max_num_seqs * (-(-(g.window + max_batched_tokens) // g.page_size) + 2)
            if g.num_pages > most:
                saved += (g.num_pages - most) * g.bytes_per_page(elem_size)
                g.num_pages = most
    keep_all = [g for g in groups if not g.window]
    if keep_all and saved:
        extra = saved // sum(g.bytes_per_page(elem_size) for g in keep_all)
        for g in keep_all:
            g.num_pages += int(extra)


class CacheStorage:
    def __init__(self, groups: list[CacheGroup], call_state_specs, num_state_slots: int,
                 dtype: torch.dtype, device):
        self.groups = groups
        self.dtype = dtype
        self.pools = []
        self._slot_home: dict[int, tuple] = {}
        for gi, g in enumerate(groups):
            if g.num_pages <= 0:
                raise ValueError(f"cache group {gi} has no pages")
            s = g.spec
            # Zeroed once and never cleared when pages are given back: correctness rests on
            # context lengths and masks, never on page contents (crates/model/src/paged.rs:53-60).
            pool = torch.zeros((len(g.slots), 2, g.num_pages, s.n_kv_heads, g.page_size, s.head_dim),
                               dtype=dtype, device=device)
            self.pools.append(pool)
            for i, slot in enumerate(g.slots):
                self._slot_home[slot] = (gi, i)
        self.states = []
        for spec in call_state_specs:
            if spec is None:
                self.states.append(None)
            else:
                self.states.append(torch.zeros((num_state_slots,) + tuple(spec.shape),
                                               dtype=spec.dtype, device=device))

    def layer_cache(self, slot: int):
        if slot not in self._slot_home:
            return None
        gi, i = self._slot_home[slot]
        return LayerCache(self.pools[gi][i, 0], self.pools[gi][i, 1], gi, self.groups[gi].page_size)

    def bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.pools)
