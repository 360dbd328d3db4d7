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

The tensors are made here; the bookkeeping (free lists, block tables, lengths, slots) is kept by
the C++ host runtime ``csrc/host_runtime.cpp``, which also packs a whole step in one call
(``bwh_pack_step``, used by the engine).  Requests are named by any hashable id here and by a
small integer handle there.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import FixedStateRequest, PagedKVRequest
from .pages import OutOfPages

_c_int_p = ctypes.POINTER(ctypes.c_int)
_c_ll_p = ctypes.POINTER(ctypes.c_longlong)
ERR_NO_SLOT, ERR_OUT_OF_PAGES, ERR_BAD_ARG, ERR_WINDOW_RELEASED = -1, -2, -3, -4
ERR_BAD_TOKEN, ERR_BAD_WANT, ERR_TOO_SMALL, ERR_TOO_MANY_TOKENS, ERR_TWICE = -5, -6, -7, -8, -9
_INVARIANTS = {-20: "a page is held twice", -21: "a page or a slot is lost (held + free != pool)",
               -22: "a held page is on the free list", -23: "a page or a slot was freed twice"}
_lib = None


def native():
    """The C++ host runtime (csrc/host_runtime.cpp), built with the host compiler at first use."""
    global _lib
    if _lib is None:
        from ..kernels.build import load_host_library
        lib = load_host_library("host_runtime")
        vp, ci, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        sigs = {"bwh_create": (vp, [ci, _c_int_p, _c_int_p, ci, ci]), "bwh_destroy": (None, [vp]),
                "bwh_add_request": (ci, [vp]), "bwh_slot": (ci, [vp, ci]), "bwh_length": (ll, [vp, ci]),
                "bwh_free_slots": (ci, [vp]), "bwh_free_pages": (ci, [vp, _c_int_p]),
                "bwh_pages_needed": (ci, [vp, ci, ll, _c_int_p]), "bwh_append": (ll, [vp, ci, ll]),
                "bwh_pages_needed_many": (ci, [vp, ci, vp, ll, _c_int_p]),
                "bwh_release_passed": (ci, [vp, ci]), "bwh_truncate": (ci, [vp, ci, ll]),
                "bwh_free_request": (ci, [vp, ci]), "bwh_num_blocks": (ci, [vp, ci, ci]),
                "bwh_blocks": (ci, [vp, ci, ci, vp, ci]), "bwh_check": (ci, [vp]),
                "bwh_pack_step": (ll, [vp, ci, vp, vp, vp, vp, vp, ci, ci, ll, vp, ll, vp, vp]),
                "bwh_release_passed_many": (ci, [vp, ci, vp])}
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


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
    pool: Optional[torch.Tensor] = None


class _Slots:
    """The free state slots, as the host runtime counts them."""

    def __init__(self, manager):
        self._m = manager

    @property
    def num_free(self) -> int:
        return native().bwh_free_slots(self._m._h)


class CacheManager:
    """The tensors (page pools, state) and the Python face of the bookkeeping, which itself lives
    in the C++ host runtime: free lists, block tables, lengths and slots."""

    def __init__(self, requests: Sequence[object], page_size: int, num_pages: int | Sequence[int],
                 max_requests: int, dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None):
        """``requests``: per schedule entry what it owns (PagedKVRequest,
        FixedStateRequest or None).  ``num_pages``: pages of each group (one number
        for all, or one per group in order of first appearance).  ``device=None``
        keeps the bookkeeping only (no tensors), for tests without a GPU."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if max_requests <= 0:
            raise ValueError("need at least one request slot")
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
                    self.groups.append(_Group(rq, [], 0))
                self.groups[by_key[rq]].entries.append(pos)
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(self.groups):
            raise ValueError(f"{len(self.groups)} cache groups but {len(counts)} page counts")
        for g, (grp, n) in enumerate(zip(self.groups, counts)):
            if n <= 0:
                raise ValueError("a page pool needs at least one page")
            grp.num_pages = int(n)
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
        G = len(self.groups)
        windows = (ctypes.c_int * max(G, 1))(*[int(g.request.window or 0) for g in self.groups])
        pages = (ctypes.c_int * max(G, 1))(*[g.num_pages for g in self.groups])
        self._h = native().bwh_create(G, windows, pages, page_size, max_requests)
        if not self._h:
            raise ValueError("the host runtime refused the cache sizes")
        self._handles: Dict[object, int] = {}
        self._scratch = (ctypes.c_int * max(G, 1))()
        self.slots = _Slots(self)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.bwh_destroy(h)

    # ------------------------------------------------------------------ requests
    def has(self, rid) -> bool:
        return rid in self._handles

    def handle(self, rid) -> int:
        """The host runtime's number for the request (-1: not live)."""
        return self._handles.get(rid, -1)

    def length(self, rid) -> int:
        return int(native().bwh_length(self._h, self._handles[rid]))

    def slot(self, rid) -> int:
        return native().bwh_slot(self._h, self._handles[rid])

    @property
    def live(self):
        return list(self._handles)

    def zero_state(self, slot: int) -> None:
        for sv in self._states:
            if sv.state is not None:
                sv.state[slot].zero_()

    def adopt(self, rid, handle: int) -> None:
        """Records a request that the host runtime created inside a packed step."""
        self._handles[rid] = handle

    def add_request(self, rid) -> int:
        """Hands the request a state slot (zeroed).  Raises if none is free."""
        if rid in self._handles:
            raise ValueError(f"request {rid!r} is already live")
        h = native().bwh_add_request(self._h)
        if h < 0:
            raise OutOfPages(f"all {self.max_requests} request slots are taken")
        self._handles[rid] = h
        slot = native().bwh_slot(self._h, h)
        self.zero_state(slot)
        return slot

    def pages_needed(self, rid, n_new: int) -> List[int]:
        """Pages each group must still hand out for the request to grow by ``n_new``."""
        if native().bwh_pages_needed(self._h, self._handles[rid], n_new, self._scratch) != 0:
            raise ValueError(f"request {rid!r} cannot grow by {n_new}")
        return list(self._scratch[:len(self.groups)])

    def pages_needed_many(self, rids, n_new: int) -> List[int]:
        """Pages each group must still hand out for every one of the requests to grow by ``n_new``."""
        hs = np.fromiter((self._handles[r] for r in rids), dtype=np.int32)
        if native().bwh_pages_needed_many(self._h, len(hs), hs.ctypes.data, n_new, self._scratch) != 0:
            raise ValueError(f"the requests cannot grow by {n_new}")
        return list(self._scratch[:len(self.groups)])

    def can_append(self, rid, n_new: int) -> bool:
        return all(n <= f for n, f in zip(self.pages_needed(rid, n_new), self.free_pages()))

    def append(self, rid, n_new: int) -> int:
        """Grows the request by ``n_new`` tokens; returns its old length.  Either
        every group hands out the pages or nothing changes and OutOfPages is raised."""
        if n_new <= 0:
            raise ValueError("a request grows by at least one token")
        old = native().bwh_append(self._h, self._handles[rid], n_new)
        if old == ERR_OUT_OF_PAGES:
            raise OutOfPages(f"request {rid!r} needs {self.pages_needed(rid, n_new)} more pages, "
                             f"{self.free_pages()} are free")
        if old < 0:
            raise ValueError(f"request {rid!r} cannot grow by {n_new} (code {old})")
        return int(old)

    def release_passed(self, rid) -> int:
        """Gives back the pages that every later query's window has passed.
        Returns how many pages were freed."""
        n = native().bwh_release_passed(self._h, self._handles[rid])
        if n < 0:
            raise AssertionError(f"release_passed({rid!r}): code {n}: {_INVARIANTS.get(n, 'bad request')}")
        return n

    def release_passed_many(self, rids) -> int:
        """:meth:`release_passed` for every request of a step, in one call."""
        if not any(g.request.window for g in self.groups):
            return 0
        hs = np.fromiter((self._handles[r] for r in rids), dtype=np.int32)
        n = native().bwh_release_passed_many(self._h, len(hs), hs.ctypes.data)
        if n < 0:
            raise AssertionError(f"release_passed: code {n}: {_INVARIANTS.get(n, 'bad request')}")
        return n

    def truncate(self, rid, new_length: int) -> None:
        """Rolls the request back to ``new_length`` tokens and gives back the pages
        behind it (the reference's rewind, src/core/paging/paged_kv_cache.h:196-208).
        Not possible into a stretch whose pages a window has already released."""
        h = self._handles[rid]
        length = int(native().bwh_length(self._h, h))
        if not 0 <= new_length <= length:
            raise ValueError(f"cannot truncate request {rid!r} of {length} tokens to {new_length}")
        if self._states and 0 < new_length < length:
            raise ValueError("a request with fixed-size state can only be rolled back to its start")
        rc = native().bwh_truncate(self._h, h, new_length)
        if rc == ERR_WINDOW_RELEASED:
            raise ValueError(f"request {rid!r}: the pages before position {new_length} were released "
                             f"by the window and cannot be restored")
        if rc != 0:
            raise AssertionError(f"truncate({rid!r}, {new_length}): code {rc}: {_INVARIANTS.get(rc, 'bad argument')}")
        if self._states and new_length == 0:
            self.zero_state(native().bwh_slot(self._h, h))

    def free_request(self, rid) -> None:
        h = self._handles.pop(rid)
        rc = native().bwh_free_request(self._h, h)
        if rc < 0:
            raise AssertionError(f"free_request({rid!r}): code {rc}: {_INVARIANTS.get(rc, 'bad request')}")

    def num_blocks(self, rid, group: int) -> int:
        """Entries of the block table of (request, group), released ones included."""
        n = native().bwh_num_blocks(self._h, self._handles[rid], group)
        if n < 0:
            raise ValueError(f"no group {group}")
        return n

    def block_row(self, rid, group: int) -> np.ndarray:
        """The block table of (request, group): int32 page ids, -1 where a window gave the page back."""
        h = self._handles[rid]
        n = native().bwh_num_blocks(self._h, h, group)
        if n < 0:
            raise ValueError(f"no group {group}")
        out = np.empty(n, dtype=np.int32)
        if n:
            native().bwh_blocks(self._h, h, group, out.ctypes.data, n)
        return out

    def block_table(self, rid, group: int) -> List[int]:
        return self.block_row(rid, group).tolist()

    # ------------------------------------------------------------------ accounting
    def free_pages(self) -> List[int]:
        native().bwh_free_pages(self._h, self._scratch)
        return list(self._scratch[:len(self.groups)])

    def check_invariants(self) -> None:
        """No page lost and none held twice: per group, pages held by requests plus
        free pages are exactly the pool; every slot is either free or a live request's."""
        rc = native().bwh_check(self._h)
        if rc != 0:
            raise AssertionError(f"cache invariants: {_INVARIANTS.get(rc, f'code {rc}')}")
        for gi, g in enumerate(self.groups):
            held = [p for rid in self._handles for p in self.block_table(rid, gi) if p >= 0]
            if len(held) != len(set(held)) or len(held) + self.free_pages()[gi] != g.num_pages:
                raise AssertionError(f"group {gi}: {len(held)} held ({len(set(held))} distinct) + "
                                     f"{self.free_pages()[gi]} free != {g.num_pages}")
