"""Cache manager: pages of keys and values with a block table per request (C++ bookkeeping in
csrc/host/kvcache.h), groups of layers with pages of their own, per-request state slots, and
the device storage behind them."""

from .host import host
from .storage import CacheGroup, CacheStorage, plan_groups, size_groups


def make_cache_manager(groups, num_state_slots: int):
    h = host()
    return h.CacheManager([h.GroupConfig(g.num_pages, g.page_size, g.window) for g in groups],
                          num_state_slots)
