"""Paged key/value cache, block tables and per-request state slots."""
from .manager import CacheManager, KVLayerView, StateLayerView
from .native_pages import NativePageTables
from .pages import NO_PAGE, CacheError, GroupSpec, PagePool, PageTables, RequestPages, SlotPool

__all__ = ["CacheManager", "KVLayerView", "StateLayerView", "NativePageTables", "NO_PAGE", "CacheError", "GroupSpec", "PagePool",
           "PageTables", "RequestPages", "SlotPool"]
