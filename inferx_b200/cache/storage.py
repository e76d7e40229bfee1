"""Device memory behind the cache manager's bookkeeping.

Per layer with a paged need: one tensor ``[pages, kv_heads, page_size, head_dim]``
(or the entry's own head size, where the need gives one) for each entry of the need (keys and values for attention; whatever a mixer names),
indexed by the page ids of the layer's group (the reference's per-layer views are
``[P, B, kv_heads, hd]``, include/inferx/core/kv_cache.h:40-150; heads are moved
outward here so that one head's part of a page is contiguous).  Per state need of a
mixer: one tensor ``[slots, *shape]``.  Everything starts from zero; a slot is zeroed again when it
is handed to a new request.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.base import LayerCache, PagedKvNeed, StateNeed
from .manager import CacheManager, is_paged_need, span_key


class CacheStorage:
    def __init__(self, cache_needs_per_layer, manager: CacheManager, dtype: torch.dtype, device):
        self.manager = manager
        self.device = torch.device(device)
        self.paged: Dict[int, Dict[str, torch.Tensor]] = {}
        self.group_of_layer: Dict[int, int] = {}
        self.state: Dict[int, Dict[str, torch.Tensor]] = {}
        span_to_group = {(g.window, getattr(g, "keep_first", 0)): i
                         for i, g in enumerate(manager.groups)}
        for layer, needs in enumerate(cache_needs_per_layer):
            for need in needs:
                if is_paged_need(need):
                    g = span_to_group[span_key(need)]
                    if self.group_of_layer.setdefault(layer, g) != g:
                        raise TypeError(f"layer {layer}: paged needs with different windows; "
                                        "one block table addresses a layer's pages")
                    pages = manager.pools[g].num_pages
                    dims = getattr(need, "entry_dims", None)
                    per = self.paged.setdefault(layer, {})
                    for i, name in enumerate(getattr(need, "entries", ("k", "v"))):
                        if name in per:
                            raise TypeError(f"layer {layer}: paged entry {name!r} named twice")
                        shape = (pages, need.kv_heads, manager.page_size,
                                 need.head_dim if dims is None else int(dims[i]))
                        per[name] = torch.zeros(shape, dtype=getattr(need, "dtype", None) or dtype,
                                                device=self.device)
                elif isinstance(need, StateNeed) or hasattr(need, "shape"):
                    self.state.setdefault(layer, {})[need.name] = torch.zeros(
                        (manager.max_slots,) + tuple(need.shape), dtype=need.dtype,
                        device=self.device)
                else:
                    raise TypeError(f"layer {layer}: unknown cache need {need!r}")

    def bytes(self) -> int:
        n = 0
        for per in self.paged.values():
            n += sum(t.numel() * t.element_size() for t in per.values())
        for per in self.state.values():
            n += sum(t.numel() * t.element_size() for t in per.values())
        return n

    def layer_caches(self, schedule, unit_of=None) -> List[LayerCache]:
        """One ``LayerCache`` per schedule entry.  ``unit_of(entry)`` gives the index of the
        entry's cache among the needs this storage was built from (the layer it names,
        when absent)."""
        out = []
        for e in schedule:
            src = unit_of(e) if unit_of is not None else e.cache_layer
            out.append(LayerCache(
                group=self.group_of_layer.get(src, -1), pages=self.paged.get(src, {}),
                writes=e.writes_cache, state=self.state.get(src, {})))
        return out

    def unit_cache(self, unit: int) -> LayerCache:
        """The cache of one unit by its index among the needs (for a part that is not a
        layer of the schedule: the embedding's state, say)."""
        return LayerCache(group=self.group_of_layer.get(unit, -1), pages=self.paged.get(unit, {}),
                          writes=True, state=self.state.get(unit, {}))

    def zero_slots(self, slots) -> None:
        if not slots:
            return
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        for per in self.state.values():
            for t in per.values():
                t.index_fill_(0, idx, 0)
