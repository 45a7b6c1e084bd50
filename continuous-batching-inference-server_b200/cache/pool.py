"""Device memory of the cache: pages per group of layers, fixed-size state per request slot.

Layers whose mixers need the same kind of cache (the same named arrays per token and the same
window) form a group; a group has one pool of pages and one block table per request,
and every layer of the group has its own arrays (attention: K and V) indexed by the same page ids
(the reference has this one implicit group: ``k_base(l)``/``v_base(l)`` share the page id,
include/paged_kv_cache.hpp:38-39; and allocates 2 L separate buffers,
src/paged_kv_cache.cpp:8-14 - here a group is one allocation).  The host bookkeeping
(free lists, block tables, slots) is the native ``CacheManager``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..kernels.library import host
from ..parts import CacheNeed


@dataclass
class LayerCache:
    """The pages of one layer: per declared array a tensor ``[num_pages, heads, page_size, width]``."""
    group: int
    arrays: Dict[str, torch.Tensor]
    page_size: int
    window: int

    @property
    def k(self) -> torch.Tensor:
        return self.arrays["k"]

    @property
    def v(self) -> torch.Tensor:
        return self.arrays["v"]


@dataclass
class CacheGroup:
    need: CacheNeed
    layers: List[int]
    page_size: int
    num_pages: int
    storage: Optional[torch.Tensor] = None   # one flat allocation: [layer][array][page][head][token][width]

    def bytes_per_page(self, itemsize: int) -> int:
        return len(self.layers) * self.need.elements_per_token() * self.page_size * itemsize


def cache_groups_of(model, page_size: int) -> List[CacheGroup]:
    groups: List[CacheGroup] = []
    for li, layer in enumerate(model.layers):
        need = layer.mixer.cache_need()
        if need is None or layer.spec.cache_source is not None:
            continue
        for g in groups:
            if g.need == need:
                g.layers.append(li)
                break
        else:
            groups.append(CacheGroup(need, [li], page_size, 0))
    return groups


class CachePool:
    def __init__(self, model, *, page_size: int = 16, num_pages: Optional[int] = None, max_requests: int = 16,
                 max_tokens: Optional[int] = None, memory_fraction: float = 0.85, device="cuda"):
        """``num_pages`` per group, or ``max_tokens`` (pages = ceil(max_tokens / page_size)), or what
        ``memory_fraction`` of the free device memory holds."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.model, self.page_size, self.max_requests = model, page_size, max_requests
        self.dtype, self.device = model.dtype, torch.device(device)
        self.groups = cache_groups_of(model, page_size)
        itemsize = torch.empty((), dtype=self.dtype).element_size()
        if num_pages is None and max_tokens is not None:
            num_pages = -(-max_tokens // page_size)
        if num_pages is None:
            free, _ = torch.cuda.mem_get_info(self.device)
            per_page = sum(g.bytes_per_page(itemsize) for g in self.groups) or 1
            num_pages = max(1, int(free * memory_fraction) // per_page)
            # no request can use more than max_requests * max_positions tokens
            num_pages = min(num_pages, max_requests * (-(-model.spec.max_positions // page_size)))
        self.layer_cache: Dict[int, LayerCache] = {}
        specs = []
        align = 256 // itemsize                      # every array starts on a 256-byte boundary (TMA wants 16)
        for gi, g in enumerate(self.groups):
            g.num_pages = int(num_pages)
            sizes = [(-(-g.num_pages * a.heads * page_size * a.width // align) * align) for a in g.need.arrays]
            g.storage = torch.zeros(len(g.layers) * sum(sizes), dtype=self.dtype, device=self.device)
            at = 0
            for li in g.layers:
                arrays = {}
                for a, size in zip(g.need.arrays, sizes):
                    n = g.num_pages * a.heads * page_size * a.width
                    arrays[a.name] = g.storage[at:at + n].view(g.num_pages, a.heads, page_size, a.width)
                    at += size
                self.layer_cache[li] = LayerCache(gi, arrays, page_size, g.need.window)
            specs.append(host().GroupSpec(page_size, g.num_pages, g.need.window))
        if not specs:  # a model without any cache still needs request slots
            specs.append(host().GroupSpec(page_size, 0, 0))
        for li, layer in enumerate(model.layers):
            src = layer.spec.cache_source
            if src is not None:
                if src not in self.layer_cache:
                    raise ValueError(f"layer {li} reads the cache of layer {src}, which keeps none")
                self.layer_cache[li] = self.layer_cache[src]
        self.manager = host().CacheManager(specs, max_requests)
        # fixed-size per-request state
        self.state: Dict[int, torch.Tensor] = {}
        for li, layer in enumerate(model.layers):
            need = layer.mixer.state_need()
            if need is not None:
                self.state[li] = torch.zeros((max_requests, *need.shape), dtype=need.dtype, device=self.device)

    def max_blocks(self, gi: int) -> int:
        return -(-self.model.spec.max_positions // self.page_size)

    def clear_state(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()

    def bytes_per_token(self) -> int:
        itemsize = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.layers) * g.need.elements_per_token() * itemsize for g in self.groups)

    def poison_pages(self, group: int, pages: Sequence[int]) -> None:
        """Fills the given pages of every array of every layer of ``group`` with NaN (a debugging aid: a
        kernel that reads a page its request no longer holds, or a token slot beyond a request's length
        inside a page that was used before, then shows up as NaN logits)."""
        if not pages or group >= len(self.groups):
            return
        idx = torch.tensor(sorted(set(int(p) for p in pages)), dtype=torch.long, device=self.device)
        for li in self.groups[group].layers:
            for t in self.layer_cache[li].arrays.values():
                t.index_fill_(0, idx, float("nan"))
