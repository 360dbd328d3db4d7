"""The cache manager: pages of keys and values with a block table per request,
and slots for per-request state of fixed size.

Layers are put into *groups* by what they need (number of kv heads, head size,
window).  Each group has its own page pool, its own free list and, per request,
its own block table; a page id indexes the same page in every layer of its group
(as one page id does across all layers in the reference,
src/core/paging/paged_kv_cache.h:74-78,96-107).  A pool is one tensor
``[entries, 2, num_pages, num_kv_heads, page_size, head_dim]`` (2: keys, values).

A request gets pages when it grows (:meth:`CacheManager.append`, all or nothing
across all groups), gives back the pages that a window has passed
(:meth:`release_passed`), and gives back everything, its state slot included,
when it ends (:meth:`free_request`).  Fixed-size state lives beside the pages in
tensors ``[max_requests, *shape]`` indexed by the request's slot and is zeroed
when the slot is handed out (the shape of the reference's SSM state pool,
src/core/ssm/ssm_state_pool.h:69-146).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import FixedStateRequest, PagedKVRequest
from .pages import OutOfPages, PageAllocator, SlotAllocator


@dataclass
class PagedKVView:
    """What a mixer sees of its cache: the pages of its schedule entry."""
    group: int
    k_pages: Optional[torch.Tensor]  # [num_pages, num_kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor]
    page_size: int


@dataclass
class StateView:
    """Per-request state of fixed size: ``state[slot]`` belongs to one request."""
    state: Optional[torch.Tensor]  # [max_requests, *shape]


@dataclass
class _Group:
    request: PagedKVRequest
    entries: List[int]
    num_pages: int
    allocator: PageAllocator
    pool: Optional[torch.Tensor] = None


@dataclass
class _Request:
    slot: int
    length: int = 0
    # per group: block table (page id, or -1 once given back) and first block still held
    blocks: List[List[int]] = field(default_factory=list)
    first_live: List[int] = field(default_factory=list)
    # int32 mirrors of `blocks` (with spare capacity), so that packing a step's batch is a memory copy
    mirrors: List[np.ndarray] = field(default_factory=list)

    def sync_mirror(self, gi: int, start: int = 0) -> None:
        """Copies blocks[gi][start:] into the mirror, growing it if needed."""
        n = len(self.blocks[gi])
        m = self.mirrors[gi]
        if n > m.shape[0]:
            grown = np.full(max(n, 2 * m.shape[0], 64), -1, dtype=np.int32)
            grown[:start] = m[:start]
            self.mirrors[gi] = m = grown
        if n > start:
            m[start:n] = self.blocks[gi][start:n]


class CacheManager:
    def __init__(self, requests: Sequence[object], page_size: int, num_pages: int | Sequence[int],
                 max_requests: int, dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None):
        """``requests``: per schedule entry what it owns (PagedKVRequest,
        FixedStateRequest or None).  ``num_pages``: pages of each group (one number
        for all, or one per group in order of first appearance).  ``device=None``
        keeps the bookkeeping only (no tensors), for tests without a GPU."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = device
        self.groups: List[_Group] = []
        self.views: List[object] = [None] * len(requests)
        self._states: List[StateView] = []
        by_key: Dict[PagedKVRequest, int] = {}
        for pos, rq in enumerate(requests):
            if isinstance(rq, PagedKVRequest):
                if rq not in by_key:
                    by_key[rq] = len(self.groups)
                    self.groups.append(_Group(rq, [], 0, None))
                self.groups[by_key[rq]].entries.append(pos)
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(self.groups):
            raise ValueError(f"{len(self.groups)} cache groups but {len(counts)} page counts")
        for g, (grp, n) in enumerate(zip(self.groups, counts)):
            grp.num_pages = n
            grp.allocator = PageAllocator(n)
            r = grp.request
            if device is not None:
                grp.pool = torch.zeros((len(grp.entries), 2, n, r.num_kv_heads, page_size, r.head_dim),
                                       dtype=dtype, device=device)
            for i, pos in enumerate(grp.entries):
                self.views[pos] = PagedKVView(g, None if grp.pool is None else grp.pool[i, 0],
                                              None if grp.pool is None else grp.pool[i, 1], page_size)
        for pos, rq in enumerate(requests):
            if isinstance(rq, FixedStateRequest):
                st = None if device is None else torch.zeros((max_requests, *rq.shape), dtype=rq.dtype,
                                                             device=device)
                self.views[pos] = StateView(st)
                self._states.append(self.views[pos])
            elif rq is not None and not isinstance(rq, PagedKVRequest):
                raise TypeError(f"schedule entry {pos}: unknown cache request {rq!r}")
        self.slots = SlotAllocator(max_requests)
        self._requests: Dict[object, _Request] = {}

    # ------------------------------------------------------------------ requests
    def has(self, rid) -> bool:
        return rid in self._requests

    def length(self, rid) -> int:
        return self._requests[rid].length

    def slot(self, rid) -> int:
        return self._requests[rid].slot

    @property
    def live(self):
        return list(self._requests)

    def add_request(self, rid) -> int:
        """Hands the request a state slot (zeroed).  Raises if none is free."""
        if rid in self._requests:
            raise ValueError(f"request {rid!r} is already live")
        slot = self.slots.try_allocate()
        if slot is None:
            raise OutOfPages(f"all {self.max_requests} request slots are taken")
        for sv in self._states:
            if sv.state is not None:
                sv.state[slot].zero_()
        self._requests[rid] = _Request(slot, 0, [[] for _ in self.groups], [0] * len(self.groups),
                                       [np.full(64, -1, dtype=np.int32) for _ in self.groups])
        return slot

    def _first_needed_block(self, grp: _Group, q_start: int) -> int:
        w = grp.request.window
        if w is None:
            return 0
        return max(0, q_start - w + 1) // self.page_size

    def pages_needed(self, rid, n_new: int) -> List[int]:
        """Pages each group must still hand out for the request to grow by ``n_new``."""
        rq = self._requests[rid]
        total = -(-(rq.length + n_new) // self.page_size)
        return [max(0, total - len(b)) for b in rq.blocks]

    def can_append(self, rid, n_new: int) -> bool:
        return all(n <= g.allocator.num_free for n, g in zip(self.pages_needed(rid, n_new), self.groups))

    def append(self, rid, n_new: int) -> int:
        """Grows the request by ``n_new`` tokens; returns its old length.  Either
        every group hands out the pages or nothing changes and OutOfPages is raised."""
        if n_new <= 0:
            raise ValueError("a request grows by at least one token")
        rq = self._requests[rid]
        need = self.pages_needed(rid, n_new)
        for n, g in zip(need, self.groups):
            if n > g.allocator.num_free:
                raise OutOfPages(f"request {rid!r} needs {n} more pages, {g.allocator.num_free} are free")
        for gi, (n, g) in enumerate(zip(need, self.groups)):
            if n:
                had = len(rq.blocks[gi])
                rq.blocks[gi].extend(g.allocator.allocate(n))
                rq.sync_mirror(gi, had)
        old = rq.length
        rq.length += n_new
        return old

    def release_passed(self, rid) -> int:
        """Gives back the pages that every later query's window has passed.
        Returns how many pages were freed."""
        rq = self._requests[rid]
        freed = 0
        for gi, g in enumerate(self.groups):
            if g.request.window is None:
                continue
            keep_from = self._first_needed_block(g, rq.length)  # the next query sits at position length
            first = rq.first_live[gi]
            if keep_from > first:
                pages = [p for p in rq.blocks[gi][first:keep_from] if p >= 0]
                g.allocator.free(pages)
                for i in range(first, keep_from):
                    rq.blocks[gi][i] = -1
                rq.mirrors[gi][first:keep_from] = -1
                rq.first_live[gi] = keep_from
                freed += len(pages)
        return freed

    def truncate(self, rid, new_length: int) -> None:
        """Rolls the request back to ``new_length`` tokens and gives back the pages
        behind it (the reference's rewind, src/core/paging/paged_kv_cache.h:196-208).
        Not possible into a stretch whose pages a window has already released."""
        rq = self._requests[rid]
        if not 0 <= new_length <= rq.length:
            raise ValueError(f"cannot truncate request {rid!r} of {rq.length} tokens to {new_length}")
        if self._states and 0 < new_length < rq.length:
            raise ValueError("a request with fixed-size state can only be rolled back to its start")
        if self._states and new_length == 0:
            for sv in self._states:
                if sv.state is not None:
                    sv.state[rq.slot].zero_()
        keep = -(-new_length // self.page_size)
        for gi, g in enumerate(self.groups):
            if g.request.window is not None and rq.first_live[gi] > self._first_needed_block(g, new_length):
                raise ValueError(f"request {rid!r}: the pages before position {new_length} were released "
                                 f"by the window and cannot be restored")
        for gi, g in enumerate(self.groups):
            tail = rq.blocks[gi][keep:]
            g.allocator.free([p for p in tail if p >= 0])
            del rq.blocks[gi][keep:]
            rq.first_live[gi] = min(rq.first_live[gi], keep)
        rq.length = new_length

    def free_request(self, rid) -> None:
        rq = self._requests.pop(rid)
        for gi, g in enumerate(self.groups):
            g.allocator.free([p for p in rq.blocks[gi] if p >= 0])
        self.slots.free(rq.slot)

    def block_table(self, rid, group: int) -> List[int]:
        return self._requests[rid].blocks[group]

    def block_row(self, rid, group: int) -> np.ndarray:
        """The same as an int32 array (a view: valid until the request changes)."""
        rq = self._requests[rid]
        return rq.mirrors[group][:len(rq.blocks[group])]

    # ------------------------------------------------------------------ accounting
    def free_pages(self) -> List[int]:
        return [g.allocator.num_free for g in self.groups]

    def held_pages(self) -> List[int]:
        return [sum(1 for r in self._requests.values() for p in r.blocks[gi] if p >= 0)
                for gi in range(len(self.groups))]

    def check_invariants(self) -> None:
        """No page lost and none held twice: per group, pages held by requests plus
        free pages are exactly the pool."""
        for gi, g in enumerate(self.groups):
            held = [p for r in self._requests.values() for p in r.blocks[gi] if p >= 0]
            if len(held) != len(set(held)):
                raise AssertionError(f"group {gi}: a page is held twice")
            if len(held) + g.allocator.num_free != g.num_pages:
                raise AssertionError(f"group {gi}: {len(held)} held + {g.allocator.num_free} free "
                                     f"!= {g.num_pages}")
            if any(g.allocator._is_free[p] for p in held):
                raise AssertionError(f"group {gi}: a held page is on the free list")
