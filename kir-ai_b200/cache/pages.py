"""Page pools, per-request block tables and fixed-size state slots (host side).

Keys and values live in pages of ``page_size`` tokens.  Layers with the same
need (kv heads, head size, window) form a group; a group has its own pool of
page ids and every request has one block table per group, shared by the
group's layers: logical page ``p`` of a request holds positions
``[p * page_size, (p + 1) * page_size)``.  Pages go back to the pool when a
request ends, and, in a windowed group, as soon as every position of a page has
fallen out of the window of all tokens still to come.  Pages are not cleared:
kernels mask by position, so stale rows are never read.

The reference keeps one contiguous ring per request and layer, capacity
``min(tokens, sliding_window)`` (crates/llm-kv-cache/src/layer.rs:390-451,765-805,
crates/llm-backend/src/core/qwen/ops/cache.rs:116-121); its free-list allocator
``BlockPool`` (crates/llm-kv-cache/src/block_pool.rs:158-171,630-670,740-760)
is the model for the pool here, without prefix sharing or copy-on-write.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

NO_PAGE = -1


class CacheError(RuntimeError):
    """Misuse of the cache manager (double free, unknown request and the like)."""


class PagePool:
    """``num_pages`` page ids with a free-list stack; a page is held by one owner."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages
        self.high_water = 0
        self.handed_out = 0  # pages given out since creation; more than num_pages means that pages were used again

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, count: int) -> Optional[List[int]]:
        """``count`` pages, or None (and nothing taken) when fewer are free."""
        if count < 0:
            raise CacheError("cannot allocate a negative number of pages")
        if count > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            if self._held[page]:
                raise CacheError(f"page {page} was on the free list while held")
            self._held[page] = True
        self.high_water = max(self.high_water, self.used_pages)
        self.handed_out += count
        return pages

    def release(self, pages: List[int]) -> None:
        for page in pages:
            if not 0 <= page < self.num_pages:
                raise CacheError(f"page id {page} is outside the pool of {self.num_pages}")
            if not self._held[page]:
                raise CacheError(f"page {page} freed twice")
            self._held[page] = False
            self._free.append(page)


class SlotPool:
    """Slots for per-request state of fixed size (position, sampler state, and the
    state tensors of mixers that ask for one)."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise CacheError(f"a slot pool needs at least one slot, got {num_slots}")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def allocate(self) -> Optional[int]:
        if not self._free:
            return None
        slot = self._free.pop()
        self._held[slot] = True
        return slot

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise CacheError(f"slot {slot} freed twice or never held")
        self._held[slot] = False
        self._free.append(slot)


@dataclass
class GroupSpec:
    """What the layers of one group keep: sizes, and the window (None = all)."""

    kv_heads: int
    head_dim: int
    window: Optional[int]
    layers: List[int] = field(default_factory=list)  # cache-layer ids in this group


@dataclass(eq=False)
class RequestPages:
    """What one live request holds: a slot, its length, one block table per group."""

    request_id: object
    slot: int
    length: int = 0  # tokens whose keys and values are in the cache
    tables: List[List[int]] = field(default_factory=list)  # per group; NO_PAGE where given back
    closed: bool = False
    version: int = 0  # bumped whenever a table changes (lets callers keep array copies of the tables)

    def pages_held(self, group: int) -> List[int]:
        return [page for page in self.tables[group] if page != NO_PAGE]


class PageTables:
    """Host bookkeeping of all groups' pools and all live requests' block tables."""

    def __init__(self, groups: List[GroupSpec], page_size: int, num_pages: List[int] | int, num_slots: int):
        if page_size <= 0:
            raise CacheError(f"page_size must be positive, got {page_size}")
        self.page_size = page_size
        self.groups = groups
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(groups)
        if len(num_pages) != len(groups):
            raise CacheError("one page count per group is needed")
        self.pools = [PagePool(n) for n in num_pages]
        self.slots = SlotPool(num_slots)
        self.live: Dict[object, RequestPages] = {}

    # -- requests ---------------------------------------------------------
    def open(self, request_id) -> Optional[RequestPages]:
        """Admits a request: a slot and empty block tables; None when no slot is free."""
        if request_id in self.live:
            raise CacheError(f"request {request_id!r} is already live")
        slot = self.slots.allocate()
        if slot is None:
            return None
        request = RequestPages(request_id, slot, 0, [[] for _ in self.groups])
        self.live[request_id] = request
        return request

    def pages_needed(self, request: RequestPages, new_tokens: int) -> List[int]:
        """Pages each group must add so that ``new_tokens`` more tokens fit."""
        total = -(-(request.length + new_tokens) // self.page_size)
        return [max(0, total - len(table)) for table in request.tables]

    def can_reserve(self, request: RequestPages, new_tokens: int) -> bool:
        need = self.pages_needed(request, new_tokens)
        return all(n <= pool.free_pages for n, pool in zip(need, self.pools))

    def reserve(self, request: RequestPages, new_tokens: int) -> bool:
        """Gives the request the pages for its next ``new_tokens`` tokens in every
        group, or nothing at all (False) when some group has too few free pages."""
        if request.closed:
            raise CacheError(f"request {request.request_id!r} is closed")
        if new_tokens < 0:
            raise CacheError("new_tokens must not be negative")
        need = self.pages_needed(request, new_tokens)
        if not all(n <= pool.free_pages for n, pool in zip(need, self.pools)):
            return False
        for table, n, pool in zip(request.tables, need, self.pools):
            if n:
                pages = pool.allocate(n)
                assert pages is not None
                table.extend(pages)
                request.version += 1
        return True

    def commit(self, request: RequestPages, new_tokens: int) -> None:
        """Records that ``new_tokens`` tokens were written, and gives back the pages
        of windowed groups that no later token can see: page p is free once
        ``(p + 1) * page_size <= length - window + 1``."""
        if request.closed:
            raise CacheError(f"request {request.request_id!r} is closed")
        new_length = request.length + new_tokens
        for table in request.tables:
            if new_length > len(table) * self.page_size:
                raise CacheError(
                    f"request {request.request_id!r}: {new_length} tokens do not fit its {len(table)} pages"
                )
        request.length = new_length
        for group, table, pool in zip(self.groups, request.tables, self.pools):
            if group.window is None:
                continue
            first_visible = request.length - group.window + 1  # lowest position a later token reads
            if first_visible <= 0:
                continue
            dead = min(first_visible // self.page_size, len(table))
            stale = [table[p] for p in range(dead) if table[p] != NO_PAGE]
            if stale:
                pool.release(stale)
                for p in range(dead):
                    table[p] = NO_PAGE
                request.version += 1

    def close(self, request: RequestPages) -> None:
        """Gives back everything the request holds (pages of every group, the slot)."""
        if request.closed:
            raise CacheError(f"request {request.request_id!r} closed twice")
        for group_index, pool in enumerate(self.pools):
            pool.release(request.pages_held(group_index))
            request.tables[group_index] = []
        request.version += 1
        self.slots.release(request.slot)
        request.closed = True
        del self.live[request.request_id]

    # -- accounting -------------------------------------------------------
    def check_consistency(self) -> None:
        """Every page is either free or held by exactly one live request."""
        for group_index, pool in enumerate(self.pools):
            seen = set()
            for request in self.live.values():
                for page in request.pages_held(group_index):
                    if page in seen:
                        raise CacheError(f"group {group_index}: page {page} held twice")
                    seen.add(page)
            if len(seen) != pool.used_pages:
                raise CacheError(
                    f"group {group_index}: {pool.used_pages} pages out of the pool, {len(seen)} in block tables"
                )
            if set(pool._free) & seen:
                raise CacheError(f"group {group_index}: a held page is on the free list")

    def stats(self) -> dict:
        return {
            "page_size": self.page_size,
            "groups": [
                {"window": g.window, "layers": len(g.layers), "pages": p.num_pages, "used": p.used_pages, "high_water": p.high_water,
                 "handed_out": p.handed_out}
                for g, p in zip(self.groups, self.pools)
            ],
            "slots_free": self.slots.free_slots,
            "live_requests": len(self.live),
        }
