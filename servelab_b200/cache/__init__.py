"""Paged key/value cache and per-request state slots."""

from .manager import (CacheError, CacheManager, FixedStateRequest, PagedKVRequest,
                      PagePool, StateSlotPool)

__all__ = ["CacheError", "CacheManager", "FixedStateRequest", "PagedKVRequest",
           "PagePool", "StateSlotPool"]
