"""The cache manager: pages, block tables and state slots, on the host.

In the manner of the reference's BlockManager (src/block_manager.h:25-57,
src/block_manager.cpp:21-59) and of how its engine uses it (src/engine.cpp:146-174):
fixed-size pages with a reference count each, handed out low ids first, one block
table per request; a request gets pages one at a time until its table covers the tokens
it is about to run and keeps what it got when the pool runs dry; all pages go back
when the request ends or is preempted.  The reference's prefix cache (hash chain, LRU
of unreferenced pages) is left out; the reference count and a ``fork`` stay.

Beyond the reference:
  * layer groups.  Layers with different needs (every key; a window of the last W keys)
    form groups, each with a pool and a block table per request of its own.  A window
    group gives a page back as soon as no later query can reach into it.
  * state slots.  A pool of slots of fixed size, one per live request (the reference's
    requests carry no device state; here the slot holds the request's logits fingerprint
    and serves mixers that keep state of their own).
Nothing in this file touches a device; storage lives in cache/storage.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

FREED = -1  # table entry of a page that a window has passed


class CacheError(RuntimeError):
    pass


class PagePool:
    """Reference-counted pages of one group."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise CacheError("a pool cannot have a negative number of pages")
        self.num_pages = num_pages
        self._ref = [0] * num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() hands out low ids first

    def available(self) -> int:
        return len(self._free)

    def allocate(self) -> Optional[int]:
        if not self._free:
            return None
        p = self._free.pop()
        self._ref[p] = 1
        return p

    def fork(self, page: int) -> None:
        if self._ref[page] <= 0:
            raise CacheError(f"fork of page {page}, which nobody holds")
        self._ref[page] += 1

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages) or self._ref[page] <= 0:
            raise CacheError(f"release of page {page}, which nobody holds")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return self._ref[page]


@dataclass(frozen=True)
class GroupSpec:
    """Layers whose caches live and die together: ``window`` None keeps every key."""
    window: Optional[int]
    entries: tuple  # cache entries (layer runs) of this group


@dataclass
class RequestCache:
    tables: List[List[int]]           # per group: page ids by block index (FREED where passed)
    first_live: List[int]             # per group: first block index not yet given back
    length: int = 0                   # tokens whose keys/values are in the cache
    slot: int = -1
    epoch: int = 0                    # goes up when the tables are emptied: entries seen before are void


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], pages_per_group: Sequence[int], page_size: int,
                 num_slots: int):
        if page_size <= 0:
            raise CacheError("page size must be positive")
        if len(groups) != len(pages_per_group):
            raise CacheError("one page count per group is needed")
        self.groups = list(groups)
        self.page_size = page_size
        self.pools = [PagePool(n) for n in pages_per_group]
        self.num_slots = num_slots
        self._free_slots = list(range(num_slots - 1, -1, -1))
        self.requests: Dict[Hashable, RequestCache] = {}

    # -- requests ----------------------------------------------------------------------
    def begin(self, rid: Hashable) -> RequestCache:
        """Register a request: an empty table per group and a state slot."""
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise CacheError("no free state slot (more live requests than slots)")
        rc = RequestCache(tables=[[] for _ in self.groups], first_live=[0] * len(self.groups),
                          slot=self._free_slots.pop())
        self.requests[rid] = rc
        return rc

    def has(self, rid: Hashable) -> bool:
        return rid in self.requests

    def get(self, rid: Hashable) -> RequestCache:
        try:
            return self.requests[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def length(self, rid: Hashable) -> int:
        return self.get(rid).length

    def ensure(self, rid: Hashable, tokens: int) -> bool:
        """Make every group's table cover positions 0 .. tokens-1.  Pages are taken one
        at a time; on failure what was gained is kept (src/engine.cpp:146-153) and False
        is returned."""
        rc = self.get(rid)
        need = (tokens + self.page_size - 1) // self.page_size
        for g, table in enumerate(rc.tables):
            while len(table) < need:
                p = self.pools[g].allocate()
                if p is None:
                    return False
                table.append(p)
        return True

    def pages_needed(self, rid: Hashable, tokens: int) -> List[int]:
        """How many more pages each group would need to cover ``tokens`` positions."""
        rc = self.get(rid)
        need = (tokens + self.page_size - 1) // self.page_size
        return [max(0, need - len(t)) for t in rc.tables]

    def advance(self, rid: Hashable, length: int) -> None:
        """Record that ``length`` tokens are now cached; window groups give back the pages
        that no later query can reach: the next query sits at position >= length and reads
        keys from ``length - window + 1`` on."""
        rc = self.get(rid)
        if length < rc.length:
            raise CacheError(f"request {rid!r}: length goes back from {rc.length} to {length}")
        if length > min((len(t) for t in rc.tables), default=0) * self.page_size and rc.tables:
            raise CacheError(f"request {rid!r}: {length} tokens exceed the pages it holds")
        rc.length = length
        for g, spec in enumerate(self.groups):
            if spec.window is None:
                continue
            first_needed = length - spec.window + 1
            table = rc.tables[g]
            while rc.first_live[g] < len(table) and (rc.first_live[g] + 1) * self.page_size <= first_needed:
                b = rc.first_live[g]
                self.pools[g].release(table[b])
                table[b] = FREED
                rc.first_live[g] += 1

    def release(self, rid: Hashable, keep_slot: bool = False) -> None:
        """Give back every page of the request (finish, cancel, preemption:
        src/engine.cpp:155-164) and, unless ``keep_slot``, its state slot."""
        rc = self.get(rid)
        for g, table in enumerate(rc.tables):
            for p in table:
                if p != FREED:
                    self.pools[g].release(p)
            table.clear()
            rc.first_live[g] = 0
        rc.length = 0
        rc.epoch += 1
        if not keep_slot:
            self._free_slots.append(rc.slot)
            del self.requests[rid]

    def fork(self, src: Hashable, dst: Hashable) -> RequestCache:
        """A new request sharing every page of ``src`` (reference counts go up)."""
        a = self.get(src)
        b = self.begin(dst)
        for g, table in enumerate(a.tables):
            for p in table:
                if p != FREED:
                    self.pools[g].fork(p)
            b.tables[g] = list(table)
            b.first_live[g] = a.first_live[g]
        b.length = a.length
        return b

    # -- bookkeeping -------------------------------------------------------------------
    def available(self, group: int = 0) -> int:
        return self.pools[group].available()

    def min_available(self) -> int:
        return min(p.available() for p in self.pools) if self.pools else 0

    def all_free(self) -> bool:
        return all(p.available() == p.num_pages for p in self.pools) and len(self._free_slots) == self.num_slots

    def free_slots(self) -> int:
        return len(self._free_slots)

    def max_blocks(self, group: int) -> int:
        return max((len(rc.tables[group]) for rc in self.requests.values()), default=0)

    def check_consistency(self) -> None:
        """No page lost, none held twice without a matching count, none both free and held."""
        for g, pool in enumerate(self.pools):
            held: Dict[int, int] = {}
            for rc in self.requests.values():
                for p in rc.tables[g]:
                    if p != FREED:
                        held[p] = held.get(p, 0) + 1
            free = set(pool._free)
            if len(free) != len(pool._free):
                raise CacheError(f"group {g}: a page is on the free list twice")
            for p in range(pool.num_pages):
                if pool.refcount(p) != held.get(p, 0):
                    raise CacheError(f"group {g}: page {p} has count {pool.refcount(p)} but {held.get(p, 0)} holders")
                if (p in free) != (pool.refcount(p) == 0):
                    raise CacheError(f"group {g}: page {p} is {'free' if p in free else 'missing'} with count "
                                     f"{pool.refcount(p)}")
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.num_slots:
            raise CacheError("a state slot is lost")


def groups_from_needs(needs: Sequence[object]) -> List[GroupSpec]:
    """Group cache entries by what must be kept: entries with paged keys and the same
    window share a group (and so a block table); entries without paged keys form none."""
    from ..parts.base import PagedKVNeed
    by_window: Dict[Optional[int], List[int]] = {}
    for e, need in enumerate(needs):
        if isinstance(need, PagedKVNeed):
            by_window.setdefault(need.window, []).append(e)
    keys = sorted(by_window, key=lambda w: (w is not None, w or 0))
    return [GroupSpec(w, tuple(by_window[w])) for w in keys]
