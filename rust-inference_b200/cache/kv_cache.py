"""The cache: a slot per sequence, keys and values per layer in pages, fixed-size
state per sequence beside them.

Layers with the same needs (kv heads, head size, window) form a *group* with
pools and a page table of its own, so that, say, full-attention layers and
sliding-window layers neither share pages nor waste them.  Pools are laid out
[entries of the group, pages, kv_heads, page_size, head_dim] (one layer's slice
is the reference's layout, thanhauco/rust-inference src/kvcache.rs:40-50).
A mixer that asks for fixed-size state gets a tensor [slots, *shape], zeroed
whenever a slot is given out.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import CacheRequest
from .allocator import CacheError, HostCache, PageTable

PAGE_SIZE = 32          # tokens per page, as in the reference (src/kvcache.rs:12)


@dataclass
class LayerCache:
    """What one scheduled layer gets: its slice of the pools, its group's page
    table, its state, and whether it appends."""
    k_pool: Optional[torch.Tensor]
    v_pool: Optional[torch.Tensor]
    page_table: Optional[torch.Tensor]
    page_size: int
    state: Optional[torch.Tensor]
    writes: bool = True


class _Group:
    def __init__(self, req: CacheRequest, entries: List[int], pages: PageTable, num_slots, num_pages,
                 max_pages_per_seq, page_size, dtype, device):
        self.req, self.entries = req, entries
        self.pages = pages
        shape = (len(entries), num_pages, req.kv_heads, page_size, req.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.table_dev = torch.full((num_slots, max_pages_per_seq), -1, dtype=torch.int32, device=device)

    def upload(self) -> None:
        pt = self.pages
        dirty = pt.take_dirty()
        if not len(dirty):
            return
        if pt.table.nbytes <= (1 << 20) or len(dirty) * 4 >= pt.num_slots:
            self.table_dev.copy_(torch.from_numpy(pt.table.copy()))
        else:
            for s in dirty.tolist():
                self.table_dev[s].copy_(torch.from_numpy(pt.table[s].copy()))


class Cache:
    """``requests[i]`` is what cache entry i's mixer asked for (None: nothing)."""

    def __init__(self, requests: Sequence[Optional[CacheRequest]], num_slots: int, num_pages: int,
                 max_pages_per_seq: int, dtype: torch.dtype, device, page_size: int = PAGE_SIZE):
        self.device = torch.device(device)
        self.dtype = dtype
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_pages_per_seq = min(max_pages_per_seq, num_pages)
        self.requests = list(requests)
        self.groups: List[_Group] = []
        self._where: Dict[int, tuple] = {}
        by_need: Dict[tuple, List[int]] = {}
        for i, r in enumerate(self.requests):
            if r is not None and r.kv_heads > 0:
                by_need.setdefault((r.kv_heads, r.head_dim, r.window), []).append(i)
        # the bookkeeping of slots, pages and lengths is one C++ object (csrc/host_cache.cpp)
        self.host = HostCache(num_slots, num_pages, self.max_pages_per_seq, page_size,
                              [need[2] for need in by_need])
        self.slots = self.host.slots
        self._any_window = any(need[2] > 0 for need in by_need)
        for (need, entries), pages in zip(by_need.items(), self.host.groups):
            g = _Group(self.requests[entries[0]], entries, pages, num_slots, num_pages, self.max_pages_per_seq,
                       page_size, dtype, self.device)
            for j, e in enumerate(entries):
                self._where[e] = (len(self.groups), j)
            self.groups.append(g)
        self.state: Dict[int, torch.Tensor] = {}
        for i, r in enumerate(self.requests):
            if r is not None and r.state_shape:
                self.state[i] = torch.zeros((num_slots,) + tuple(r.state_shape), dtype=r.state_dtype, device=self.device)

    # ---- slots ---------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        s = self.host.alloc_slot()
        for t in self.state.values():
            t[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.host.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.host.length(slot)

    @property
    def max_seq_len(self) -> int:
        return self.max_pages_per_seq * self.page_size

    def free_pages(self) -> int:
        return self.host.free_pages()

    # ---- growth ----------------------------------------------------------------------------
    def extend(self, growth: Sequence[tuple]) -> List[int]:
        """``growth``: (slot, new_tokens) for every sequence of a step.  Maps the
        pages in every group and returns each sequence's length before.  Either
        all of it happens or none."""
        return self.host.extend([g[0] for g in growth], [g[1] for g in growth])

    def upload(self) -> None:
        """Bring the device page tables up to date (before the step's kernels)."""
        for g in self.groups:
            g.upload()

    def after_step(self, slots: Sequence[int]) -> None:
        """Release what no later step can read (pages behind a window)."""
        if self._any_window:
            self.host.after_step(slots)

    # ---- views -----------------------------------------------------------------------------
    def layer(self, entry: int, writes: bool = True) -> LayerCache:
        state = self.state.get(entry)
        if entry in self._where:
            gi, j = self._where[entry]
            g = self.groups[gi]
            return LayerCache(g.k[j], g.v[j], g.table_dev, self.page_size, state, writes)
        return LayerCache(None, None, None, self.page_size, state, writes)

    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.entries) * g.req.kv_heads * g.req.head_dim * es for g in self.groups)

    def check(self) -> None:
        self.host.check()
