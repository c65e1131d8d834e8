"""The cache manager: pages of keys/values per layer group, and state slots.

Host-side bookkeeping only (no tensors; ``cache/storage.py`` owns the device
memory).  Layers whose mixers have the same cache needs form a *group*; each
group has its own pool of pages and its own block table per request:

  * a full-attention group keeps every page of a request until it ends;
  * a windowed group (window w) gives a page back as soon as every key in it is
    out of reach of all future queries; the table keeps a -1 in its place so
    that logical page i still sits at index i;
  * a fixed-state group holds no pages: the request's *state slot* indexes a
    fixed-size record per layer.  The slot pool exists even when no layer asks
    for state, and is taken and returned with the pages.

Pages leave the free list at the left and return at the right (FIFO reuse,
deterministic), as in the reference's BlockManager (servelab/kv_cache/
manager.py:42,187-189,226).  Growing is ``ensure`` (allocate_slots/append_slot,
manager.py:153-202), giving back is ``release`` (manager.py:216-227), the slot
formula is table[p // bs] * bs + p % bs (manager.py:309-313; evaluated on the
device here).  Prefix matching, swap and offload are not part of this engine.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple


# ------------------------------------------------------------ what mixers ask
@dataclass(frozen=True)
class PagedKVRequest:
    """Keys and values of ``num_kv_heads`` x ``head_dim`` per token, paged.
    ``window`` None: all earlier tokens stay readable; else only the last
    ``window`` positions (the current one included)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedStateRequest:
    """A per-request record of fixed ``shape`` (float32) in a state slot."""
    shape: Tuple[int, ...]


class CacheError(RuntimeError):
    pass


# ------------------------------------------------------------------ one group
class PagePool:
    """Pages of one layer group and the block tables that point into them."""

    def __init__(self, num_pages: int, page_size: int, window: Optional[int] = None):
        if num_pages < 1 or page_size < 1:
            raise ValueError("num_pages and page_size must be >= 1")
        self.num_pages = num_pages
        self.page_size = page_size
        self.window = window
        self.free: deque = deque(range(num_pages))
        self.tables: Dict[str, List[int]] = {}
        self._first_live: Dict[str, int] = {}
        self._serial = 0                       # bumped whenever any table changes
        self.stamp: Dict[str, int] = {}        # request -> serial of its table's last change
        # called with the pages that return to the free list (a request ended, a window passed them)
        self.on_free: Optional[Callable[[List[int]], None]] = None

    def num_free(self) -> int:
        return len(self.free)

    def pages_for(self, num_tokens: int) -> int:
        return -(-num_tokens // self.page_size)

    def new_pages_needed(self, req: str, num_tokens: int) -> int:
        return max(0, self.pages_for(num_tokens) - len(self.tables[req]))

    def peak_pages(self, total_tokens: int, max_portion: int) -> int:
        """Most pages a request of ``total_tokens`` can hold at once when fed in
        portions of at most ``max_portion`` tokens."""
        full = self.pages_for(total_tokens)
        if self.window is None:
            return full
        return min(full, self.pages_for(self.window + max_portion) + 1)

    def open(self, req: str) -> None:
        if req in self.tables:
            raise CacheError(f"request {req} already has a block table")
        self.tables[req] = []
        self._first_live[req] = 0
        self._touch(req)

    def _touch(self, req: str) -> None:
        self._serial += 1
        self.stamp[req] = self._serial

    def grow(self, req: str, num_tokens: int) -> List[int]:
        need = self.new_pages_needed(req, num_tokens)
        if need > len(self.free):
            raise CacheError("grow() without enough free pages")
        new = [self.free.popleft() for _ in range(need)]
        if new:
            self.tables[req].extend(new)
            self._touch(req)
        return new

    def trim(self, req: str, next_position: int) -> List[int]:
        """Give back pages no query at position >= ``next_position`` can read."""
        if self.window is None:
            return []
        table = self.tables[req]
        # keys needed: r >= next_position - window + 1
        dead_pages = max(0, (next_position - self.window + 1) // self.page_size)
        dead_pages = min(dead_pages, len(table))
        freed = []
        for lp in range(self._first_live[req], dead_pages):
            if table[lp] >= 0:
                freed.append(table[lp])
                table[lp] = -1
        self._first_live[req] = max(self._first_live[req], dead_pages)
        self.free.extend(freed)
        if freed:
            self._touch(req)
            if self.on_free is not None:
                self.on_free(freed)
        return freed

    def close(self, req: str) -> List[int]:
        table = self.tables.pop(req, None)
        self._first_live.pop(req, None)
        self.stamp.pop(req, None)
        if table is None:
            return []
        freed = [p for p in table if p >= 0]
        self.free.extend(freed)
        if freed and self.on_free is not None:
            self.on_free(freed)
        return freed


class StateSlotPool:
    """Slots for per-request state of fixed size; a slot must be cleared by the
    device side before its first use, so freshly taken slots are queued."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self.free: deque = deque(range(num_slots))
        self.owner: Dict[str, int] = {}
        self.to_clear: List[int] = []

    def num_free(self) -> int:
        return len(self.free)

    def take(self, req: str) -> Optional[int]:
        if req in self.owner:
            raise CacheError(f"request {req} already holds a state slot")
        if not self.free:
            return None
        slot = self.free.popleft()
        self.owner[req] = slot
        self.to_clear.append(slot)
        return slot

    def give(self, req: str) -> Optional[int]:
        slot = self.owner.pop(req, None)
        if slot is not None:
            self.free.append(slot)
        return slot

    def drain_to_clear(self) -> List[int]:
        out, self.to_clear = self.to_clear, []
        return out


# ---------------------------------------------------------------- all groups
class CacheManager:
    """All groups' pools plus the state slots; requests are opened, grown,
    trimmed and released across every group at once (all or nothing)."""

    def __init__(self, group_windows: Sequence[Optional[int]], num_pages, page_size: int,
                 num_state_slots: int, reserve_pages: int = 0):
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(group_windows)
        if len(num_pages) != len(group_windows):
            raise ValueError("one page count per group is needed")
        self.page_size = page_size
        self.pools = [PagePool(n, page_size, w) for n, w in zip(num_pages, group_windows)]
        self.slots = StateSlotPool(num_state_slots)
        self.reserve_pages = reserve_pages
        self.alloc_fails = 0
        # called with the request's id whenever a request gives everything back (it ended,
        # was aborted or preempted): whoever keeps copies of its tables drops them
        self.release_listeners: List[Callable[[str], None]] = []

    # ------------------------------------------------------------- queries
    def has(self, req: str) -> bool:
        return req in self.slots.owner

    def block_table(self, req: str, group: int) -> List[int]:
        return self.pools[group].tables[req]

    def state_slot(self, req: str) -> int:
        return self.slots.owner[req]

    def table_stamp(self, req: str, group: int) -> int:
        """A number that changes whenever the request's table in that group changes
        (unique across requests of the group), so callers can cache copies."""
        return self.pools[group].stamp[req]

    def can_ever_hold(self, total_tokens: int, max_portion: int) -> bool:
        return all(p.peak_pages(total_tokens, max_portion) <= p.num_pages - self.reserve_pages
                   for p in self.pools)

    def can_grow(self, req: Optional[str], num_tokens: int, for_admission: bool = False) -> bool:
        hold_back = self.reserve_pages if for_admission else 0
        for p in self.pools:
            need = p.pages_for(num_tokens) if req is None else p.new_pages_needed(req, num_tokens)
            if need > p.num_free() - hold_back:
                return False
        return True

    # ----------------------------------------------------------- mutations
    def open(self, req: str) -> bool:
        """Take a state slot and create empty tables; False if no slot is free."""
        if self.slots.take(req) is None:
            return False
        for p in self.pools:
            p.open(req)
        return True

    def ensure(self, req: str, num_tokens: int, for_admission: bool = False) -> bool:
        """Make room for the request's first ``num_tokens`` tokens in every
        group, or change nothing and return False."""
        if not self.can_grow(req, num_tokens, for_admission):
            self.alloc_fails += 1
            return False
        for p in self.pools:
            p.grow(req, num_tokens)
        return True

    def trim(self, req: str, next_position: int) -> None:
        for p in self.pools:
            p.trim(req, next_position)

    def release(self, req: str) -> None:
        """Give back every page of every group and the state slot; harmless for
        an unknown request."""
        for p in self.pools:
            p.close(req)
        self.slots.give(req)
        for listener in self.release_listeners:
            listener(req)

    # --------------------------------------------------------------- stats
    def stats(self) -> dict:
        return {
            "pages_free": [p.num_free() for p in self.pools],
            "pages_used": [p.num_pages - p.num_free() for p in self.pools],
            "slots_free": self.slots.num_free(),
            "alloc_fails": self.alloc_fails,
        }

    def usage(self) -> float:
        total = sum(p.num_pages for p in self.pools)
        return (total - sum(p.num_free() for p in self.pools)) / max(1, total)

    def check_invariants(self) -> None:
        """Every page is either free or in exactly one table; same for slots."""
        for gi, p in enumerate(self.pools):
            seen = list(p.free)
            for table in p.tables.values():
                seen.extend(x for x in table if x >= 0)
            if sorted(seen) != list(range(p.num_pages)):
                lost = set(range(p.num_pages)) - set(seen)
                twice = {x for x in seen if seen.count(x) > 1}
                raise CacheError(f"group {gi}: pages lost {sorted(lost)}, held twice {sorted(twice)}")
        seen = list(self.slots.free) + list(self.slots.owner.values())
        if sorted(seen) != list(range(self.slots.num_slots)):
            raise CacheError("state slots lost or held twice")
        for p in self.pools:
            if set(p.tables) != set(self.slots.owner):
                raise CacheError("tables and slots disagree on live requests")
