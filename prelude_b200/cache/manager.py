"""The cache manager: paged keys and values, block tables, state slots.

Each entry of a model's run order states what its cache must hold
(``KvPagesNeed``, ``StateNeed`` or nothing).  Entries with the same need (heads,
head size, window) form a *group*; a group has a page pool, an allocator and,
for every live request, a block table of its own, so layers that keep all keys
and layers that keep a window of them never share pages.  Entries with a
``StateNeed`` get one tensor of ``max_slots`` fixed-size states; every request
holds one slot for its whole life, whether or not any layer uses it.

Pages are taken when a request's token count grows (``grow``), given back when
a window has passed them (``trim``) and when the request ends (``release``),
and are then used again by whoever asks next.  The reference keeps one pool
with per-layer tensors [pages, page_size, heads, head_dim]; here a page is laid out
head by head, [pages, heads, page_size, head_dim], so that the keys (or values) of one head in one page
are one contiguous run of memory, which is what the attention kernels fetch at a time
(crates/prelude-core/src/scheduler/components/cache/manager.rs:286-329) and
declares the per-layer needs that grouping rests on
(crates/prelude-core/src/scheduler/components/cache/mod.rs:13-30).

Host bookkeeping works without a device (``device=None``), which is how the
CPU tests drive it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..engine.batch import LayerCache
from ..parts.registry import KvPagesNeed, StateNeed
from .pages import CacheAccountingError, OutOfPages, PageAllocator, SlotAllocator


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class KvGroup:
    gid: int
    need: KvPagesNeed
    members: List[int]
    allocator: PageAllocator
    k_pages: Dict[int, torch.Tensor] = field(default_factory=dict)
    v_pages: Dict[int, torch.Tensor] = field(default_factory=dict)

    def bytes_per_page(self, page_size: int, elem_size: int) -> int:
        return 2 * len(self.members) * page_size * self.need.n_kv_heads * self.need.head_dim * elem_size


@dataclass
class RequestCache:
    slot: int
    n_tokens: int = 0
    tables: Dict[int, List[int]] = field(default_factory=dict)    # group -> page ids, -1 once trimmed


class CacheManager:
    def __init__(self, needs: Sequence[object], page_size: int, num_pages: int, max_slots: int,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16,
                 max_request_tokens: Optional[int] = None):
        """``needs[n]`` is the cache need of entry n of the run order (None for
        an entry without a cache of its own).  Every group gets ``num_pages`` pages
        of ``page_size`` tokens.  With ``max_request_tokens`` every group also keeps
        its block tables on the device, one row per state slot, updated entry by
        entry (captured decode steps read those)."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.num_pages, self.max_slots = page_size, num_pages, max_slots
        self.device, self.dtype = device, dtype
        self.groups: List[KvGroup] = []
        self.group_of: Dict[int, int] = {}                 # order index -> group id
        self.state_needs: Dict[int, StateNeed] = {}
        self.state_tensors: Dict[int, torch.Tensor] = {}
        by_need: Dict[KvPagesNeed, KvGroup] = {}
        for n, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, KvPagesNeed):
                g = by_need.get(need)
                if g is None:
                    g = KvGroup(len(self.groups), need, [], PageAllocator(num_pages))
                    by_need[need] = g
                    self.groups.append(g)
                g.members.append(n)
                self.group_of[n] = g.gid
            elif isinstance(need, StateNeed):
                self.state_needs[n] = need
            else:
                raise TypeError(f"order entry {n}: unknown cache need {need!r}")
        self.slots = SlotAllocator(max_slots)
        self.requests: Dict[Hashable, RequestCache] = {}
        self._fresh_slots: List[int] = []
        self.table_width = _ceil_div(max_request_tokens, page_size) if max_request_tokens else 0
        self.device_tables: Dict[int, torch.Tensor] = {}
        # pending writes to the device-resident tables: group -> {cell (slot * width + index): page}.  A cell
        # written twice before a flush keeps its last value only, so the scatter never sees an index twice.
        self._table_updates: Dict[int, Dict[int, int]] = {}
        if self.table_width:
            for g in self.groups:
                self._table_updates[g.gid] = {}
        if device is not None:
            self._allocate_tensors()
            for g in self.groups if self.table_width else ():
                self.device_tables[g.gid] = torch.full((max_slots, self.table_width), -1, dtype=torch.int32, device=device)

    # -- device memory ----------------------------------------------------------------
    def _allocate_tensors(self) -> None:
        for g in self.groups:
            shape = (self.num_pages, g.need.n_kv_heads, self.page_size, g.need.head_dim)
            for n in g.members:
                g.k_pages[n] = torch.zeros(shape, dtype=self.dtype, device=self.device)
                g.v_pages[n] = torch.zeros(shape, dtype=self.dtype, device=self.device)
        for n, need in self.state_needs.items():
            self.state_tensors[n] = torch.zeros((self.max_slots,) + tuple(need.shape), dtype=need.dtype, device=self.device)

    @staticmethod
    def bytes_per_page(needs: Sequence[object], page_size: int, elem_size: int) -> int:
        """Device bytes that one page id costs over all groups and layers."""
        total = 0
        for need in needs:
            if isinstance(need, KvPagesNeed):
                total += 2 * page_size * need.n_kv_heads * need.head_dim * elem_size
        return total

    def layer_cache(self, n: int) -> LayerCache:
        """What entry n of the run order reads and writes."""
        if n in self.group_of:
            g = self.groups[self.group_of[n]]
            return LayerCache("kv", g.gid, g.k_pages.get(n), g.v_pages.get(n))
        if n in self.state_needs:
            return LayerCache("state", -1, state=self.state_tensors.get(n))
        return LayerCache(None)

    def layer_caches(self, n_entries: int) -> List[LayerCache]:
        return [self.layer_cache(n) for n in range(n_entries)]

    # -- requests ---------------------------------------------------------------------
    def add_request(self, rid: Hashable) -> int:
        """Register a request and give it a state slot (zeroed before its first step)."""
        if rid in self.requests:
            raise CacheAccountingError(f"request {rid!r} is already live")
        slot = self.slots.allocate()
        self.requests[rid] = RequestCache(slot, 0, {g.gid: [] for g in self.groups})
        self._fresh_slots.append(slot)
        return slot

    def has_request(self, rid: Hashable) -> bool:
        return rid in self.requests

    def tokens_of(self, rid: Hashable) -> int:
        return self.requests[rid].n_tokens

    def slot_of(self, rid: Hashable) -> int:
        return self.requests[rid].slot

    def pages_needed(self, rid: Optional[Hashable], n_tokens: int) -> Dict[int, int]:
        """New pages per group that growing request ``rid`` (None: a request not
        yet added) to ``n_tokens`` tokens would take."""
        want = _ceil_div(n_tokens, self.page_size)
        rc = self.requests.get(rid) if rid is not None else None
        return {g.gid: max(0, want - (len(rc.tables[g.gid]) if rc else 0)) for g in self.groups}

    def can_grow(self, rid: Optional[Hashable], n_tokens: int, reserve: int = 0) -> bool:
        return all(self.groups[gid].allocator.num_free - reserve >= n for gid, n in self.pages_needed(rid, n_tokens).items())

    def grow(self, rid: Hashable, n_tokens: int) -> None:
        """Make room for the request's first ``n_tokens`` tokens in every group,
        or raise OutOfPages having taken nothing."""
        rc = self.requests[rid]
        if n_tokens < rc.n_tokens:
            raise CacheAccountingError(f"request {rid!r} holds {rc.n_tokens} tokens; cannot shrink to {n_tokens}")
        need = self.pages_needed(rid, n_tokens)
        for gid, n in need.items():
            if not self.groups[gid].allocator.can_allocate(n):
                raise OutOfPages(f"request {rid!r} needs {n} more pages in cache group {gid} for {n_tokens} tokens; "
                                 f"{self.groups[gid].allocator.num_free} of {self.num_pages} are free")
        for gid, n in need.items():
            table = rc.tables[gid]
            new = self.groups[gid].allocator.allocate(n)
            for i, p in enumerate(new):
                self._queue_table_update(gid, rc.slot, len(table) + i, p)
            table.extend(new)
        rc.n_tokens = n_tokens

    def rewind(self, rid: Hashable, n_tokens: int) -> None:
        """The request holds fewer tokens than room was made for (a run of queued steps ended early): count
        ``n_tokens``; the pages stay with the request, which grows into them again."""
        rc = self.requests[rid]
        if not 0 <= n_tokens <= rc.n_tokens:
            raise CacheAccountingError(f"request {rid!r} holds {rc.n_tokens} tokens; cannot rewind to {n_tokens}")
        rc.n_tokens = n_tokens

    def trim(self, rid: Hashable) -> int:
        """Give back the pages of window groups that no later token can read.
        The next query sits at position n_tokens and reads keys from
        n_tokens - window + 1 on.  Returns the number of pages freed."""
        rc = self.requests[rid]
        freed = 0
        for g in self.groups:
            if g.need.window is None:
                continue
            first_pos = rc.n_tokens - g.need.window + 1
            if first_pos <= 0:
                continue
            table = rc.tables[g.gid]
            for i in range(min(first_pos // self.page_size, len(table))):
                if table[i] >= 0:
                    g.allocator.free([table[i]])
                    table[i] = -1
                    freed += 1
                    self._queue_table_update(g.gid, rc.slot, i, -1)
        return freed

    def _queue_table_update(self, gid: int, slot: int, index: int, page: int) -> None:
        ups = self._table_updates.get(gid)
        if ups is not None and index < self.table_width:
            ups[slot * self.table_width + index] = page

    def _drop_table_updates(self, slot: int) -> None:
        """Forget the pending writes to a slot's row: its request has ended or starts over, and what it queued
        must not land in the row once another request (or its own new start) owns it."""
        lo, hi = slot * self.table_width, (slot + 1) * self.table_width
        for ups in self._table_updates.values():
            for cell in [c for c in ups if lo <= c < hi]:
                del ups[cell]

    def take_table_updates(self) -> Dict[int, "object"]:
        """group -> int32 array [2, n] (cells; pages) of the writes that are due, each cell once; the queue is
        empty afterwards.  ``flush_table_updates`` applies them to the device-resident tables."""
        import numpy as np
        out = {}
        for gid, ups in self._table_updates.items():
            if not ups:
                continue
            arr = np.empty((2, len(ups)), dtype=np.int32)
            arr[0] = np.fromiter(ups.keys(), dtype=np.int64, count=len(ups))
            arr[1] = np.fromiter(ups.values(), dtype=np.int64, count=len(ups))
            ups.clear()
            out[gid] = arr
        return out

    def flush_table_updates(self) -> int:
        """Bring the device-resident block tables up to date; returns the number
        of entries written.  Every cell is written at most once per flush (its last
        queued value), so the scatter's threads never race.  Rows of ended requests
        keep stale entries: a kernel reads a row only up to its request's length,
        and the next owner of the slot overwrites what it reads."""
        from ..ops import kernels as K
        total = 0
        for gid, arr in self.take_table_updates().items():
            dev = torch.from_numpy(arr).to(self.device, non_blocking=True)
            K.scatter_i32(self.device_tables[gid], dev[0], dev[1])
            total += arr.shape[1]
        return total

    def release(self, rid: Hashable) -> None:
        """The request has ended: all its pages and its slot go back."""
        rc = self.requests.pop(rid, None)
        if rc is None:
            raise CacheAccountingError(f"request {rid!r} is not live")
        for g in self.groups:
            g.allocator.free([p for p in rc.tables[g.gid] if p >= 0])
        self.slots.free(rc.slot)
        self._drop_table_updates(rc.slot)
        if rc.slot in self._fresh_slots:
            self._fresh_slots.remove(rc.slot)

    def reset_request(self, rid: Hashable) -> None:
        """Drop what the request holds but keep it registered (a rolled-back or
        preempted request starts over from its first token)."""
        rc = self.requests[rid]
        for g in self.groups:
            g.allocator.free([p for p in rc.tables[g.gid] if p >= 0])
            rc.tables[g.gid] = []
        rc.n_tokens = 0
        self._drop_table_updates(rc.slot)
        if rc.slot not in self._fresh_slots:
            self._fresh_slots.append(rc.slot)

    def block_tables(self, rids: Sequence[Hashable]) -> Dict[int, List[List[int]]]:
        return {g.gid: [self.requests[r].tables[g.gid] for r in rids] for g in self.groups}

    def take_fresh_slots(self) -> List[int]:
        """Slots handed out (or reset) since the last call: their state must be
        zeroed before the next step."""
        out, self._fresh_slots = self._fresh_slots, []
        return out

    def zero_fresh_state(self) -> None:
        fresh = self.take_fresh_slots()
        if fresh and self.state_tensors:
            idx = torch.as_tensor(fresh, dtype=torch.long, device=self.device)
            for t in self.state_tensors.values():
                t.index_fill_(0, idx, 0)

    # -- accounting -------------------------------------------------------------------
    def free_pages(self) -> int:
        """Free pages in the tightest group."""
        return min((g.allocator.num_free for g in self.groups), default=self.num_pages)

    def used_pages(self) -> int:
        return max((g.allocator.num_used for g in self.groups), default=0)

    def check(self) -> None:
        """No page lost, none held twice: every group's held pages are exactly
        the pages in live block tables, each once."""
        self.slots.check()
        live_slots = sorted(rc.slot for rc in self.requests.values())
        if len(set(live_slots)) != len(live_slots):
            raise CacheAccountingError("two requests hold the same state slot")
        if self.slots.num_free + len(live_slots) != self.max_slots:
            raise CacheAccountingError("a state slot is lost")
        for g in self.groups:
            g.allocator.check()
            held: Dict[int, int] = {}
            for rc in self.requests.values():
                for p in rc.tables[g.gid]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            for p in range(self.num_pages):
                if g.allocator.refcount(p) != held.get(p, 0):
                    raise CacheAccountingError(
                        f"group {g.gid} page {p}: {g.allocator.refcount(p)} references, {held.get(p, 0)} table entries")
