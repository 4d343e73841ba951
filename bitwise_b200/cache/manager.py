"""The cache manager: pages, block tables and state slots, on the host.

The bookkeeping itself is C++ (csrc/host_runtime.cpp, reached through ``bitwise_b200.host``);
the classes here name requests by any hashable id, turn the library's error codes into
``CacheError`` and give Python views of a request's state.

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

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

from .. import host

FREED = -1  # table entry of a page that a window has passed


class CacheError(RuntimeError):
    pass


def _raise() -> None:
    raise CacheError(host.last_error())


class PagePool:
    """Reference-counted pages of one group (a pool on its own, as tests and tools use it)."""

    def __init__(self, num_pages: int):
        self._lib = host.lib()
        self._h = self._lib.bw_pool_create(num_pages)
        if not self._h:
            _raise()
        self.num_pages = num_pages

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bw_pool_destroy(self._h)
            self._h = None

    def available(self) -> int:
        return self._lib.bw_pool_available(self._h)

    def allocate(self) -> Optional[int]:
        p = self._lib.bw_pool_allocate(self._h)
        return None if p < 0 else p

    def fork(self, page: int) -> None:
        if self._lib.bw_pool_fork(self._h, page) < 0:
            _raise()

    def release(self, page: int) -> None:
        if self._lib.bw_pool_release(self._h, page) < 0:
            _raise()

    def refcount(self, page: int) -> int:
        r = self._lib.bw_pool_refcount(self._h, page)
        if r < 0:
            _raise()
        return r


@dataclass(frozen=True)
class GroupSpec:
    """Layers whose caches live and die together: ``window`` None keeps every key."""
    window: Optional[int]
    entries: tuple  # cache entries (layer runs) of this group


class RequestCache:
    """A live request's state, read from the manager on demand: ``tables`` (per group: page
    ids by block index, FREED where a window has passed), ``first_live`` (per group: first
    block not yet given back), ``length`` (tokens whose keys and values are cached), ``slot``
    and ``epoch`` (a number that no other generation of tables of this manager has had: it
    changes when the request's tables are emptied or the request begins anew)."""

    __slots__ = ("_m", "_key", "rid")

    def __init__(self, manager: "CacheManager", rid: Hashable, key: int):
        self._m, self.rid, self._key = manager, rid, key

    def _info(self):
        m = self._m
        if m._lib.bw_cm_info(m._h, self._key, m._info_buf) < 0:
            _raise()
        return m._info_buf

    @property
    def length(self) -> int:
        return self._info()[0]

    @property
    def slot(self) -> int:
        return self._info()[1]

    @property
    def epoch(self) -> int:
        return self._info()[2]

    @property
    def first_live(self) -> List[int]:
        info = self._info()
        return [info[4 + 2 * g] for g in range(self._m.num_groups)]

    def table_len(self, group: int) -> int:
        return self._info()[3 + 2 * group]

    @property
    def tables(self) -> List[List[int]]:
        m = self._m
        out = []
        for g in range(m.num_groups):
            n = self.table_len(g)
            buf = (ctypes.c_int * max(n, 1))()
            if m._lib.bw_cm_table(m._h, self._key, g, 0, buf, n, FREED) < 0:
                _raise()
            out.append(list(buf[:n]))
        return out


class _PoolView:
    """``manager.pools[g]``: what tests and tools read of one group's pool."""

    def __init__(self, manager: "CacheManager", group: int, num_pages: int):
        self._m, self._g, self.num_pages = manager, group, num_pages

    def available(self) -> int:
        return self._m.available(self._g)

    def refcount(self, page: int) -> int:
        r = self._m._lib.bw_cm_refcount(self._m._h, self._g, page)
        if r < 0:
            _raise()
        return r


class _Rows:
    def __init__(self, manager: "CacheManager", max_seqs: int):
        self._lib = manager._lib
        self._h = self._lib.bw_rows_create(max_seqs, manager.num_groups)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bw_rows_destroy(self._h)
            self._h = None


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], pages_per_group: Sequence[int], page_size: int,
                 num_slots: int):
        if page_size <= 0:
            raise CacheError("page size must be positive")
        if len(groups) != len(pages_per_group):
            raise CacheError("one page count per group is needed")
        self._lib = host.lib()
        self.groups = list(groups)
        self.num_groups = len(self.groups)
        self.page_size = page_size
        self.num_slots = num_slots
        n = self.num_groups
        windows = (ctypes.c_int * max(n, 1))(*[(-1 if g.window is None else int(g.window)) for g in self.groups])
        pages = (ctypes.c_int * max(n, 1))(*[int(p) for p in pages_per_group])
        self._h = self._lib.bw_cm_create(n, windows, pages, page_size, num_slots)
        if not self._h:
            _raise()
        self.pools = [_PoolView(self, g, int(pages_per_group[g])) for g in range(n)]
        self._info_buf = (ctypes.c_int * (3 + 2 * max(n, 1)))()
        self._need_buf = (ctypes.c_int * max(n, 1))()
        self._keys: Dict[Hashable, int] = {}   # request id -> the library's 64-bit key
        self._views: Dict[Hashable, RequestCache] = {}
        self._next_key = 1
        self._held = set()                      # ids whose keys outlive their releases

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bw_cm_destroy(self._h)
            self._h = None

    # -- requests ----------------------------------------------------------------------
    def key_of(self, rid: Hashable) -> int:
        """The library's key of a request id, given out on first sight."""
        k = self._keys.get(rid)
        if k is None:
            k = self._next_key
            self._next_key += 1
            self._keys[rid] = k
        return k

    def begin(self, rid: Hashable) -> RequestCache:
        """Register a request: an empty table per group and a state slot."""
        if rid in self._views:
            raise CacheError(f"request {rid!r} is already live")
        key = self.key_of(rid)
        if self._lib.bw_cm_begin(self._h, key) < 0:
            raise CacheError(host.last_error())
        rc = RequestCache(self, rid, key)
        self._views[rid] = rc
        return rc

    def has(self, rid: Hashable) -> bool:
        return rid in self._views

    def get(self, rid: Hashable) -> RequestCache:
        try:
            return self._views[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def length(self, rid: Hashable) -> int:
        return self.get(rid).length

    def ensure(self, rid: Hashable, tokens: int) -> bool:
        """Make every group's table cover positions 0 .. tokens-1.  Pages are taken one
        at a time; on failure what was gained is kept (src/engine.cpp:146-153) and False
        is returned."""
        r = self._lib.bw_cm_ensure(self._h, self.get(rid)._key, tokens)
        if r < 0:
            _raise()
        return r == 1

    def pages_needed(self, rid: Hashable, tokens: int) -> List[int]:
        """How many more pages each group would need to cover ``tokens`` positions."""
        if self._lib.bw_cm_pages_needed(self._h, self.get(rid)._key, tokens, self._need_buf) < 0:
            _raise()
        return [self._need_buf[g] for g in range(self.num_groups)]

    def advance(self, rid: Hashable, length: int) -> None:
        """Record that ``length`` tokens are now cached; window groups give back the pages
        that no later query can reach: the next query sits at position >= length and reads
        keys from ``length - window + 1`` on."""
        if self._lib.bw_cm_advance(self._h, self.get(rid)._key, length) < 0:
            raise CacheError(f"request {rid!r}: {host.last_error()}")

    def release(self, rid: Hashable, keep_slot: bool = False) -> None:
        """Give back every page of the request (finish, cancel, preemption:
        src/engine.cpp:155-164) and, unless ``keep_slot``, its state slot."""
        if self._lib.bw_cm_release(self._h, self.get(rid)._key, int(keep_slot)) < 0:
            _raise()
        if not keep_slot:
            self._forget(rid)

    def _forget(self, rid: Hashable) -> None:
        self._views.pop(rid, None)
        if rid not in self._held:
            self._keys.pop(rid, None)

    def hold_key(self, rid: Hashable) -> None:
        """Keep the request's key across releases (the scheduler names a request by it for as
        long as it is queued, preempted or running)."""
        self._held.add(rid)

    def drop_key(self, rid: Hashable) -> None:
        self._held.discard(rid)
        if rid not in self._views:
            self._keys.pop(rid, None)

    def sync_with_library(self, rids: Sequence[Hashable]) -> None:
        """The scheduler works on the library's side and lets requests go or takes new ones
        in there: bring this object's table of views in line for the given ids."""
        for rid in rids:
            key = self._keys.get(rid)
            live = key is not None and bool(self._lib.bw_cm_has(self._h, key))
            if live and rid not in self._views:
                self._views[rid] = RequestCache(self, rid, key)
            elif not live and rid in self._views:
                del self._views[rid]

    def fork(self, src: Hashable, dst: Hashable) -> RequestCache:
        """A new request sharing every page of ``src`` (reference counts go up)."""
        a = self.get(src)
        if dst in self._views:
            raise CacheError(f"request {dst!r} is already live")
        key = self.key_of(dst)
        if self._lib.bw_cm_fork(self._h, a._key, key) < 0:
            self._keys.pop(dst, None)
            _raise()
        rc = RequestCache(self, dst, key)
        self._views[dst] = rc
        return rc

    def snapshot(self, rid: Hashable):
        """(length, slot, epoch, table length per group, first live block per group) in one call."""
        b = self.get(rid)._info()
        n = self.num_groups
        return b[0], b[1], b[2], [b[3 + 2 * g] for g in range(n)], [b[4 + 2 * g] for g in range(n)]

    def new_rows(self, max_seqs: int) -> "_Rows":
        """The memory of what each row of a step function's block tables holds (see ``prepare_rows``)."""
        return _Rows(self, max_seqs)

    def prepare_rows(self, rows: "_Rows", n: int, keys, counts, dst_address: int, table_offsets, max_blocks,
                     starts, slots) -> int:
        """For the ``n`` requests of a step (library keys and new-token counts in ctypes arrays):
        take the pages each needs and bring its rows of the block tables, in int32 memory at
        ``dst_address``, up to date; fills ``starts`` (tokens already cached) and ``slots``.
        Returns 0; 1 + i when request i found no free page (those before it keep what they
        got); -(2 + i) when request i would outgrow its row."""
        rc = self._lib.bw_cm_prepare(self._h, rows._h, n, keys, counts, dst_address, table_offsets, max_blocks,
                                     starts, slots)
        if rc == -1:
            _raise()
        return rc

    # -- bookkeeping -------------------------------------------------------------------
    def available(self, group: int = 0) -> int:
        r = self._lib.bw_cm_available(self._h, group)
        if r < 0:
            _raise()
        return r

    def min_available(self) -> int:
        return min((self.available(g) for g in range(self.num_groups)), default=0)

    def all_free(self) -> bool:
        return bool(self._lib.bw_cm_all_free(self._h))

    def free_slots(self) -> int:
        return self._lib.bw_cm_free_slots(self._h)

    def max_blocks(self, group: int) -> int:
        r = self._lib.bw_cm_max_blocks(self._h, group)
        if r < 0:
            _raise()
        return r

    def check_consistency(self) -> None:
        """No page lost, none held twice without a matching count, none both free and held."""
        if self._lib.bw_cm_check(self._h) < 0:
            _raise()
        if self._lib.bw_cm_live(self._h) != len(self._views):
            raise CacheError("the library and its Python view disagree on the live requests")


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
