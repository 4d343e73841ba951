"""Device storage behind the cache manager's page ids and slots.

Per cache entry (layer run) keys and values are ``[pages, kv_heads, page_size,
head_dim]`` each, the reference's layout per layer (src/kernels.h:91-103;
src/model.cpp:241-248), in the dtype of the path.  A page id indexes every entry of its
group at once, as the reference's block id indexes every layer (src/model.h:69-70).
Slot state is ``[slots, *shape]`` per entry that asks for it, plus one 64-bit word per
slot for the request's logits fingerprint.  Nothing is zeroed on reuse: reads are limited
to the positions a request has written.

Behind the pages and slots that the manager hands out lies one more of each
(``pad_pages[g]``, ``pad_slot``): where the rows of a step that fills its batch up to a round
size write and read, so that they touch nothing of a request.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..parts.base import PagedKVNeed, PagedKVView, SlotStateNeed, SlotStateView
from .manager import CacheManager, GroupSpec

FINGERPRINT_SEED = 1469598103934665603  # src/engine.h:68


class CacheStorage:
    def __init__(self, needs: Sequence[object], groups: Sequence[GroupSpec], pages_per_group: Sequence[int],
                 page_size: int, num_slots: int, dtype: torch.dtype, device):
        self.needs = list(needs)
        self.groups = list(groups)
        self.page_size = page_size
        self.group_of_entry = {}
        for g, spec in enumerate(groups):
            for e in spec.entries:
                self.group_of_entry[e] = g
        self.k: List[Optional[torch.Tensor]] = [None] * len(needs)
        self.v: List[Optional[torch.Tensor]] = [None] * len(needs)
        self.state: List[Optional[torch.Tensor]] = [None] * len(needs)
        for e, need in enumerate(needs):
            if isinstance(need, PagedKVNeed):
                pages = pages_per_group[self.group_of_entry[e]]
                shape = (max(pages, 1) + 1, need.kv_heads, page_size, need.head_dim)
                self.k[e] = torch.zeros(shape, dtype=dtype, device=device)
                self.v[e] = torch.zeros(shape, dtype=dtype, device=device)
            elif isinstance(need, SlotStateNeed):
                self.state[e] = torch.zeros((max(num_slots, 1) + 1,) + tuple(need.shape), dtype=need.dtype, device=device)
            elif need is not None:
                raise TypeError(f"cache entry {e}: unknown need {need!r}")
        self.fingerprints = torch.zeros(max(num_slots, 1) + 1, dtype=torch.int64, device=device)
        self.pad_pages = [max(int(p), 1) for p in pages_per_group]  # per group: the page no request ever holds
        self.pad_slot = max(num_slots, 1)

    def nbytes(self) -> int:
        ts = [t for t in self.k + self.v + self.state if t is not None]
        return sum(t.numel() * t.element_size() for t in ts)

    def views(self, block_tables: Sequence[torch.Tensor], seq_slot: torch.Tensor) -> List[object]:
        """The per-entry views of one step: ``block_tables[g]`` is the device table of group g."""
        out: List[object] = []
        for e, need in enumerate(self.needs):
            if isinstance(need, PagedKVNeed):
                out.append(PagedKVView(self.k[e], self.v[e], block_tables[self.group_of_entry[e]], self.page_size))
            elif isinstance(need, SlotStateNeed):
                out.append(SlotStateView(self.state[e], seq_slot))
            else:
                out.append(None)
        return out


def build_cache(model, pages: int, page_size: int, num_slots: int, dtype: torch.dtype, device,
                pages_per_group: Optional[Sequence[int]] = None):
    """A manager and its storage for ``model``: ``pages`` pages in every group unless
    ``pages_per_group`` says otherwise."""
    from .manager import groups_from_needs
    needs = model.cache_needs()
    groups = groups_from_needs(needs)
    counts = list(pages_per_group) if pages_per_group is not None else [pages] * len(groups)
    manager = CacheManager(groups, counts, page_size, num_slots)
    storage = CacheStorage(needs, groups, counts, page_size, num_slots, dtype, device)
    return manager, storage
