"""The cache manager: device memory for pages and state slots over the host tables.

Cache layers with the same need share a group: one pool of page ids, one block
table per request, and one device tensor
``[layers_in_group, num_pages, 2, kv_heads, page_size, head_dim]`` (keys at index 0,
values at index 1 of the third axis), so a layer's pages are a contiguous slab
and a (page, kv head) tile is ``page_size`` contiguous rows.  Mixers with a
fixed-size state get ``[num_slots, *shape]`` per layer, zeroed when a slot is
given out.  Page memory is zeroed once at creation and never again: kernels mask
by position, so rows of an earlier owner are never read.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import KVCacheNeed, StateNeed
from .native_pages import NativePageTables
from .pages import NO_PAGE, CacheError, GroupSpec, PageTables, RequestPages


@dataclass
class KVLayerView:
    """What an attention layer sees of its cache layer."""

    kv: Optional[torch.Tensor]  # [num_pages, 2, kv_heads, page_size, head_dim]
    group: int
    page_size: int
    window: Optional[int]


@dataclass
class StateLayerView:
    """What a mixer with fixed-size state sees: ``state[slot]`` for each request of the batch."""

    state: Optional[torch.Tensor]  # [num_slots, *shape]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class CacheManager:
    def __init__(self, needs: Sequence[object], *, page_size: int, num_slots: int, dtype: torch.dtype = torch.float32,
                 device=None, num_pages: Optional[int] = None, max_tokens: Optional[int] = None, native: bool = True):
        """``needs``: one KVCacheNeed or StateNeed per cache layer.  The pool of every
        group gets ``num_pages`` pages, or enough for ``max_tokens`` tokens."""
        if num_pages is None:
            if max_tokens is None:
                raise CacheError("give num_pages or max_tokens")
            num_pages = max(1, _round_up(max_tokens, page_size) // page_size)
        self.page_size, self.num_pages, self.num_slots = page_size, num_pages, num_slots
        self.dtype, self.device = dtype, (torch.device(device) if device is not None else None)
        # a page size that the attention kernels of this dtype would refuse at the first step is refused here
        from ..csrc.ops import page_size_refusal

        for layer, need in enumerate(needs):
            if isinstance(need, KVCacheNeed):
                reason = page_size_refusal(dtype, need.head_dim, page_size)
                if reason is not None:
                    raise CacheError(f"cache layer {layer}: {reason}")
        groups: List[GroupSpec] = []
        self._layer_place: Dict[int, tuple] = {}  # cache layer -> ("kv", group, index in group) | ("state", key)
        for layer, need in enumerate(needs):
            if isinstance(need, KVCacheNeed):
                for index, group in enumerate(groups):
                    if (group.kv_heads, group.head_dim, group.window) == (need.kv_heads, need.head_dim, need.window):
                        break
                else:
                    groups.append(GroupSpec(need.kv_heads, need.head_dim, need.window))
                    index = len(groups) - 1
                self._layer_place[layer] = ("kv", index, len(groups[index].layers))
                groups[index].layers.append(layer)
            elif isinstance(need, StateNeed):
                self._layer_place[layer] = ("state", need)
            else:
                raise CacheError(f"cache layer {layer}: unknown need {need!r}")
        self.groups = groups
        # the bookkeeping runs in native code; ``native=False`` takes the Python model of the same rules
        tables_class = NativePageTables if native else PageTables
        self.tables = tables_class(groups, page_size, [num_pages] * len(groups) if groups else [], num_slots)
        self.kv: List[Optional[torch.Tensor]] = []
        self.state: Dict[int, Optional[torch.Tensor]] = {}
        for group in groups:
            shape = (len(group.layers), num_pages, 2, group.kv_heads, page_size, group.head_dim)
            self.kv.append(torch.zeros(shape, dtype=dtype, device=self.device) if self.device is not None else None)
        for layer, place in self._layer_place.items():
            if place[0] == "state":
                need = place[1]
                self.state[layer] = (
                    torch.zeros((num_slots, *need.shape), dtype=need.dtype, device=self.device)
                    if self.device is not None else None
                )

    # -- what layers see --------------------------------------------------
    def layer_view(self, layer: int):
        place = self._layer_place[layer]
        if place[0] == "kv":
            _, group, index = place
            tensor = self.kv[group][index] if self.kv[group] is not None else None
            return KVLayerView(tensor, group, self.page_size, self.groups[group].window)
        return StateLayerView(self.state[layer])

    # -- requests ---------------------------------------------------------
    def open(self, request_id) -> Optional[RequestPages]:
        request = self.tables.open(request_id)
        if request is not None:
            for tensor in self.state.values():
                if tensor is not None:
                    tensor[request.slot].zero_()
        return request

    def can_reserve(self, request: RequestPages, new_tokens: int) -> bool:
        return self.tables.can_reserve(request, new_tokens)

    def reserve(self, request: RequestPages, new_tokens: int) -> bool:
        return self.tables.reserve(request, new_tokens)

    def commit(self, request: RequestPages, new_tokens: int) -> None:
        self.tables.commit(request, new_tokens)

    def close(self, request: RequestPages) -> None:
        self.tables.close(request)

    def pages_for_tokens(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def free_pages(self) -> List[int]:
        return [pool.free_pages for pool in self.tables.pools]

    def block_table_array(self, requests: Sequence[RequestPages], group: int, min_width: int = 1) -> np.ndarray:
        """int32 [len(requests), width] of page ids, NO_PAGE where a request holds none."""
        if isinstance(self.tables, NativePageTables):
            return self.tables.fill_tables(requests, group, min_width)
        rows = [np.asarray(r.tables[group], dtype=np.int32) for r in requests]
        width = max(min_width, max((r.size for r in rows), default=0))
        array = np.full((len(requests), width), NO_PAGE, dtype=np.int32)
        for index, row in enumerate(rows):
            array[index, : row.size] = row
        return array

    def bytes_per_token(self) -> int:
        element = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.layers) * 2 * g.kv_heads * g.head_dim * element for g in self.groups)

    def stats(self) -> dict:
        return self.tables.stats()
