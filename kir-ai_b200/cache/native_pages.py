"""The page tables in native code (csrc/page_tables.cpp) behind the interface of
``pages.PageTables``.  The cache manager uses this one; the Python classes in ``pages`` stay as
the readable model, and the tests drive both with the same random sequences of requests."""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..csrc import build as _build
from .pages import NO_PAGE, CacheError, GroupSpec

_lib = None

_ERRORS = {
    -2: "unknown or closed request",
    -3: "request is already live",
    -4: "a page or slot was freed twice, or a page id is out of range",
    -5: "tokens do not fit the pages reserved for the request",
    -6: "bad argument",
}


def _library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(_build.build_host())
        lib.kirai_pages_create.restype = ctypes.c_void_p
        lib.kirai_pages_create.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_long), ctypes.c_int,
                                           ctypes.POINTER(ctypes.c_int), ctypes.c_int]
        lib.kirai_pages_destroy.argtypes = [ctypes.c_void_p]
        for name, args in {
            "kirai_pages_open": [ctypes.c_long], "kirai_pages_can_reserve": [ctypes.c_long, ctypes.c_long],
            "kirai_pages_reserve": [ctypes.c_long, ctypes.c_long], "kirai_pages_commit": [ctypes.c_long, ctypes.c_long],
            "kirai_pages_close": [ctypes.c_long], "kirai_pages_needed": [ctypes.c_long, ctypes.c_long, ctypes.POINTER(ctypes.c_int)],
            "kirai_pages_table": [ctypes.c_long, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int],
            "kirai_pages_fill_tables": [ctypes.POINTER(ctypes.c_long), ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int],
            "kirai_pages_stat": [ctypes.c_int, ctypes.c_int], "kirai_pages_check": [],
        }.items():
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_void_p, *args]
        for name in ("kirai_pages_length", "kirai_pages_version"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_long
            fn.argtypes = [ctypes.c_void_p, ctypes.c_long]
        _lib = lib
    return _lib


def _checked(code: int, what: str) -> int:
    if code < -1:
        raise CacheError(f"{what}: {_ERRORS.get(code, f'error {code}')}")
    return code


class _PoolView:
    def __init__(self, owner: "NativePageTables", group: int):
        self._owner, self._group = owner, group

    def _stat(self, what: int) -> int:
        return self._owner._lib.kirai_pages_stat(self._owner._handle, self._group, what)

    num_pages = property(lambda self: self._stat(0))
    free_pages = property(lambda self: self._stat(1))
    used_pages = property(lambda self: self._stat(2))
    high_water = property(lambda self: self._stat(3))
    handed_out = property(lambda self: self._stat(4))


class _SlotsView:
    def __init__(self, owner: "NativePageTables"):
        self._owner = owner

    num_slots = property(lambda self: self._owner._lib.kirai_pages_stat(self._owner._handle, -1, 0))
    free_slots = property(lambda self: self._owner._lib.kirai_pages_stat(self._owner._handle, -1, 1))


class NativeRequest:
    """What one live request holds, read from the native tables on demand."""

    def __init__(self, owner: "NativePageTables", request_id, key: int, slot: int):
        self._owner, self.request_id, self.key, self.slot = owner, request_id, key, slot
        self.closed = False
        self._final_length = 0
        self._cached = (-1, None)

    @property
    def length(self) -> int:
        if self.closed:
            return self._final_length
        return int(self._owner._lib.kirai_pages_length(self._owner._handle, self.key))

    @property
    def version(self) -> int:
        return -1 if self.closed else int(self._owner._lib.kirai_pages_version(self._owner._handle, self.key))

    @property
    def tables(self) -> List[List[int]]:
        if self.closed:
            return [[] for _ in self._owner.groups]
        version = self.version
        if self._cached[0] != version:
            lib, handle = self._owner._lib, self._owner._handle
            tables = []
            for group in range(len(self._owner.groups)):
                count = lib.kirai_pages_table(handle, self.key, group, None, 0)
                buffer = (ctypes.c_int * max(count, 1))()
                lib.kirai_pages_table(handle, self.key, group, buffer, count)
                tables.append(list(buffer[:count]))
            self._cached = (version, tables)
        return self._cached[1]

    def pages_held(self, group: int) -> List[int]:
        return [page for page in self.tables[group] if page != NO_PAGE]


class NativePageTables:
    def __init__(self, groups: List[GroupSpec], page_size: int, num_pages, num_slots: int):
        if page_size <= 0:
            raise CacheError(f"page_size must be positive, got {page_size}")
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(groups)
        if len(num_pages) != len(groups):
            raise CacheError("one page count per group is needed")
        if any(n <= 0 for n in num_pages):
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        if num_slots <= 0:
            raise CacheError(f"a slot pool needs at least one slot, got {num_slots}")
        self._lib = _library()
        self.page_size, self.groups = page_size, groups
        windows = (ctypes.c_long * max(len(groups), 1))(*[-1 if g.window is None else g.window for g in groups])
        counts = (ctypes.c_int * max(len(groups), 1))(*num_pages)
        self._handle = self._lib.kirai_pages_create(len(groups), windows, page_size, counts, num_slots)
        if not self._handle:
            raise CacheError("the native page tables could not be created")
        self.pools = [_PoolView(self, g) for g in range(len(groups))]
        self.slots = _SlotsView(self)
        self.live: Dict[object, NativeRequest] = {}
        self._next_key = 1

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle and self._lib is not None:
            self._lib.kirai_pages_destroy(handle)

    # -- requests ---------------------------------------------------------
    def open(self, request_id) -> Optional[NativeRequest]:
        if request_id in self.live:
            raise CacheError(f"request {request_id!r} is already live")
        key = self._next_key
        slot = _checked(self._lib.kirai_pages_open(self._handle, key), f"open {request_id!r}")
        if slot < 0:
            return None
        self._next_key += 1
        request = NativeRequest(self, request_id, key, slot)
        self.live[request_id] = request
        return request

    # -- for the native scheduler, which opens and closes requests itself ----------------------------
    def new_key(self) -> int:
        """A key that no request of these tables has had."""
        key = self._next_key
        self._next_key += 1
        return key

    def adopt(self, request_id, key: int, slot: int) -> NativeRequest:
        """The handle of a request that native code has opened under ``key``."""
        if request_id in self.live:
            raise CacheError(f"request {request_id!r} is already live")
        request = NativeRequest(self, request_id, key, slot)
        self.live[request_id] = request
        return request

    def disown(self, request: NativeRequest) -> None:
        """Marks the handle of a request that native code has closed."""
        if not request.closed:
            request.closed = True
            self.live.pop(request.request_id, None)

    def _alive(self, request: NativeRequest) -> None:
        if request.closed:
            raise CacheError(f"request {request.request_id!r} is closed")

    def pages_needed(self, request: NativeRequest, new_tokens: int) -> List[int]:
        self._alive(request)
        need = (ctypes.c_int * max(len(self.groups), 1))()
        _checked(self._lib.kirai_pages_needed(self._handle, request.key, new_tokens, need), "pages_needed")
        return list(need[: len(self.groups)])

    def can_reserve(self, request: NativeRequest, new_tokens: int) -> bool:
        self._alive(request)
        return _checked(self._lib.kirai_pages_can_reserve(self._handle, request.key, new_tokens), "can_reserve") == 1

    def reserve(self, request: NativeRequest, new_tokens: int) -> bool:
        self._alive(request)
        if new_tokens < 0:
            raise CacheError("new_tokens must not be negative")
        return _checked(self._lib.kirai_pages_reserve(self._handle, request.key, new_tokens), "reserve") == 1

    def commit(self, request: NativeRequest, new_tokens: int) -> None:
        self._alive(request)
        _checked(self._lib.kirai_pages_commit(self._handle, request.key, new_tokens), f"commit of request {request.request_id!r}")

    def close(self, request: NativeRequest) -> None:
        if request.closed:
            raise CacheError(f"request {request.request_id!r} closed twice")
        request._final_length = request.length
        _checked(self._lib.kirai_pages_close(self._handle, request.key), f"close of request {request.request_id!r}")
        request.closed = True
        del self.live[request.request_id]

    def fill_tables(self, requests: Sequence[NativeRequest], group: int, min_width: int = 1) -> np.ndarray:
        """int32 [len(requests), width] of page ids, NO_PAGE where a request holds none."""
        count = len(requests)
        keys = (ctypes.c_long * max(count, 1))(*[r.key for r in requests])
        width = min_width
        for request in requests:
            width = max(width, self._lib.kirai_pages_table(self._handle, request.key, group, None, 0))
        array = np.empty((count, width), dtype=np.int32)
        _checked(self._lib.kirai_pages_fill_tables(self._handle, keys, count, group,
                                                   array.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), width), "fill_tables")
        return array

    # -- accounting -------------------------------------------------------
    def check_consistency(self) -> None:
        code = self._lib.kirai_pages_check(self._handle)
        if code != 0:
            raise CacheError({1: "a page id in a block table is out of range", 2: "a page is held twice",
                              3: "a page is lost: pages out of the pool and pages in block tables differ",
                              4: "a held page is on the free list"}.get(code, f"check {code} failed"))

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
