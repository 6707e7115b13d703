"""The cache manager: pages of keys and values with a block table per request, in groups of
layers with the same need, and slots for per-request state of fixed size.

The reference gives every attention layer a block table of its own drawing from one pool
(src/main.zig:687-696), lets conv/SSM layers keep their state inside the layer object
(src/transformer/short_conv.zig:63-64) and frees a sequence's blocks when it finishes
(src/paged_attention/scheduler.zig:221-234, paged_kv_cache.zig:90-93).  Here:

* every entry of the model's running order that owns a cache belongs to a *group* of entries
  with the same need.  Paged groups (all keys, or a window of them) have pages of their own: one
  pool, and one block table per request; a page id addresses the same page in every member's
  plane.  State groups hold one fixed-size 32-bit state per request and member, addressed by the
  request's slot.
* pages are taken just before the step that fills them, given back when the request ends, and,
  in a window group, as soon as every position of the page has left the window.
* page 0 of every paged group and slot 0 are never handed out: padding rows of a fixed-shape
  decode batch point at them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from ..parts.base import StateNeed
from .pages import IdPool, OutOfPages

NULL_PAGE = 0
NULL_SLOT = 0
RELEASED = -1


@dataclass
class CacheGroup:
    need: object
    members: List[int] = field(default_factory=list)   # entries of the running order, in plane order
    pool: Optional[IdPool] = None                       # paged groups
    data: Optional[torch.Tensor] = None                 # device memory

    @property
    def paged(self) -> bool:
        return hasattr(self.need, "page_shape")


@dataclass
class RequestCache:
    request_id: object
    slot: int
    tables: Dict[int, List[int]]          # group index -> physical page per logical page (RELEASED if given back)
    num_tokens: int = 0                   # positions whose pages are reserved
    capacity: int = 0                     # positions that the pages held in every group cover


@dataclass
class CacheView:
    """What one layer call sees of the cache during one step."""
    group: int = -1
    pages: Optional[torch.Tensor] = None        # [num_pages, *need.page_shape(page_size)]; keys and values:
    #                                             [num_pages, 2, kv_heads, page_size, head_dim]
    block_table: Optional[torch.Tensor] = None  # [requests of the step, max pages] int32
    page_size: int = 0
    state: Optional[torch.Tensor] = None        # [slots, *shape] in the need's dtype (32-bit by default)


class CacheManager:
    def __init__(self, needs, page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype, device, allocate: bool = True):
        """`needs` is `Model.cache_needs()`: per entry of the running order ("own", its needs) or
        ("shared", the entry whose cache it reads); the needs of an entry are a tuple (a single need or
        None is taken as a tuple of one or none).  `num_pages` pages (beside the null page) are given to
        every paged group; `max_requests` slots (beside the null slot) exist."""
        if page_size < 1 or num_pages < 1 or max_requests < 1:
            raise ValueError("page_size, num_pages and max_requests should be positive")
        self.page_size, self.num_pages, self.max_requests = int(page_size), int(num_pages), int(max_requests)
        self.dtype, self.device = dtype, device
        self.groups: List[CacheGroup] = []
        self.where: List[List[tuple]] = []          # running-order entry -> [(group, plane) per need]
        by_need = {}
        for k, (how, need) in enumerate(needs):
            if how == "shared":
                self.where.append(self.where[need])
                continue
            entry = []
            for one in (() if need is None else (tuple(need) if isinstance(need, (tuple, list)) else (need,))):
                if one not in by_need:
                    by_need[one] = len(self.groups)
                    self.groups.append(CacheGroup(one))
                g = by_need[one]
                entry.append((g, len(self.groups[g].members)))
                self.groups[g].members.append(k)
            self.where.append(entry)
        for grp in self.groups:
            if grp.paged:
                grp.pool = IdPool(self.num_pages, first=1, what="page")
                if allocate:
                    grp.data = torch.zeros((len(grp.members), self.num_pages + 1) + tuple(grp.need.page_shape(self.page_size)),
                                           dtype=dtype, device=device)
            elif isinstance(grp.need, StateNeed):
                if allocate:
                    grp.data = torch.zeros((len(grp.members), self.max_requests + 1) + tuple(grp.need.shape),
                                           dtype=self._state_dtype(grp.need), device=device)
            else:
                raise TypeError(f"unknown cache need {grp.need!r}")
        self.slots = IdPool(self.max_requests, first=1, what="slot")
        # host mirror of every block table, one row per slot, ready to be gathered into a step's batch
        self._rows = {gi: np.zeros((self.max_requests + 1, 16), dtype=np.int32) for gi in self.paged_groups()}
        self._has_window = any(g.paged and g.need.window is not None for g in self.groups)
        self.requests: Dict[object, RequestCache] = {}
        self.pages_reused = 0
        self._ever_used = [set() for _ in self.groups]

    # ------------------------------------------------------------------ sizes
    def _state_dtype(self, need: StateNeed) -> torch.dtype:
        if isinstance(need.dtype, torch.dtype):
            return need.dtype
        if need.dtype == "model":
            return self.dtype
        return {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
                "int32": torch.int32}[need.dtype]

    def bytes_per_token(self) -> int:
        esize = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.members) * g.need.elements_per_token() * esize for g in self.groups if g.paged)

    def paged_groups(self):
        return [i for i, g in enumerate(self.groups) if g.paged]

    def _first_needed_page(self, grp: CacheGroup, cached: int) -> int:
        """Logical pages below this index hold no position that a query at position >= `cached`
        may still read."""
        if grp.need.window is None:
            return 0
        first_pos = max(cached - grp.need.window + 1, 0)
        return first_pos // self.page_size

    def pages_to_take(self, request_id, total_tokens: int) -> Dict[int, int]:
        """Pages each paged group would have to hand out so that the request can hold positions
        0..total_tokens-1 (counting what `reserve` would first give back)."""
        rc = self.requests[request_id]
        out = {}
        n_logical = -(-total_tokens // self.page_size)
        for gi in self.paged_groups():
            grp, table = self.groups[gi], rc.tables[gi]
            first = self._first_needed_page(grp, rc.num_tokens)
            gives_back = sum(1 for j in range(min(first, len(table))) if table[j] != RELEASED)
            takes = max(n_logical - max(len(table), first), 0)
            out[gi] = takes - gives_back
        return out

    def _fits_already(self, rc: RequestCache, total_tokens: int) -> bool:
        """True if the pages the request holds already cover `total_tokens` positions and no window
        has anything to give back (the common case of a decoded token inside its last page)."""
        if self._has_window:
            return False
        n_logical = -(-total_tokens // self.page_size)
        return all(len(t) >= n_logical for t in rc.tables.values())

    def _set_row(self, gi: int, slot: int, j: int, page: int) -> None:
        rows = self._rows[gi]
        if j >= rows.shape[1]:
            grown = np.zeros((rows.shape[0], max(2 * rows.shape[1], j + 1)), dtype=np.int32)
            grown[:, :rows.shape[1]] = rows
            self._rows[gi] = rows = grown
        rows[slot, j] = page

    def try_reserve(self, request_id, total_tokens: int) -> bool:
        """`reserve` if it is possible, in one call; False (and nothing taken) if pages are short.  The
        common case, a decoded token inside the request's last page, is a comparison."""
        rc = self.requests[request_id]
        if not self._has_window and rc.num_tokens <= total_tokens <= rc.capacity:
            rc.num_tokens = total_tokens
            return True
        if not self.can_reserve(request_id, total_tokens):
            return False
        self.reserve(request_id, total_tokens)
        return True

    def can_reserve(self, request_id, total_tokens: int) -> bool:
        if self._fits_already(self.requests[request_id], total_tokens):
            return True
        need = self.pages_to_take(request_id, total_tokens)
        return all(self.groups[gi].pool.n_free >= n for gi, n in need.items())

    def max_tokens_possible(self) -> int:
        """The longest request that could ever be held alone."""
        return self.num_pages * self.page_size

    # ------------------------------------------------------------------ life of a request
    def admit(self, request_id) -> RequestCache:
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} is already admitted")
        slot = self.slots.alloc()
        for grp in self.groups:
            if not grp.paged and grp.data is not None:
                grp.data[:, slot].zero_()
        rc = RequestCache(request_id, slot, {gi: [] for gi in self.paged_groups()})
        rc.capacity = 0 if rc.tables else 1 << 40
        self.requests[request_id] = rc
        return rc

    def reserve(self, request_id, total_tokens: int) -> None:
        """Make room for positions up to total_tokens-1.  Pages that the window has passed are
        given back first.  Takes all pages it needs or none (raises OutOfPages)."""
        rc = self.requests[request_id]
        if total_tokens < rc.num_tokens:
            raise ValueError("a request's cache does not shrink")
        if self._fits_already(rc, total_tokens):
            rc.num_tokens = total_tokens
            return
        if not self.can_reserve(request_id, total_tokens):
            raise OutOfPages(f"request {request_id!r} needs pages {self.pages_to_take(request_id, total_tokens)}, "
                             f"free {[self.groups[g].pool.n_free for g in self.paged_groups()]}")
        n_logical = -(-total_tokens // self.page_size)
        for gi in self.paged_groups():
            grp, table = self.groups[gi], rc.tables[gi]
            first = self._first_needed_page(grp, rc.num_tokens)
            for j in range(min(first, len(table))):
                if table[j] != RELEASED:
                    grp.pool.free(table[j])
                    table[j] = RELEASED
                    self._set_row(gi, rc.slot, j, NULL_PAGE)
            while len(table) < n_logical:
                if len(table) < first:
                    table.append(RELEASED)
                    continue
                p = grp.pool.alloc()
                if p in self._ever_used[gi]:
                    self.pages_reused += 1
                self._ever_used[gi].add(p)
                self._set_row(gi, rc.slot, len(table), p)
                table.append(p)
        rc.num_tokens = total_tokens
        rc.capacity = min((len(t) for t in rc.tables.values()), default=1 << 40) * self.page_size

    def release(self, request_id) -> None:
        """Give back everything the request holds."""
        rc = self.requests.pop(request_id)
        for gi, table in rc.tables.items():
            for p in table:
                if p != RELEASED:
                    self.groups[gi].pool.free(p)
            self._rows[gi][rc.slot, :] = NULL_PAGE
        self.slots.free(rc.slot)

    def check(self) -> None:
        """No page lost, held twice or freed twice; every held page belongs to exactly one request."""
        self.slots.check()
        held_slots = [rc.slot for rc in self.requests.values()]
        if len(set(held_slots)) != len(held_slots) or set(held_slots) != set(self.slots._refs):
            raise AssertionError("slots and requests disagree")
        for gi in self.paged_groups():
            pool = self.groups[gi].pool
            pool.check()
            owned = [p for rc in self.requests.values() for p in rc.tables[gi] if p != RELEASED]
            if len(set(owned)) != len(owned):
                raise AssertionError("a page is in two block tables")
            if set(owned) != set(pool._refs):
                raise AssertionError("held pages and block tables disagree")

    def stats(self) -> dict:
        out = {"slots_used": self.slots.n_used, "slots_free": self.slots.n_free,
               "slots_high_water": self.slots.high_water, "pages_reused": self.pages_reused}
        for gi in self.paged_groups():
            pool = self.groups[gi].pool
            out[f"group{gi}_pages_used"] = pool.n_used
            out[f"group{gi}_pages_free"] = pool.n_free
            out[f"group{gi}_pages_high_water"] = pool.high_water
        return out

    # ------------------------------------------------------------------ what a step sees
    def table_rows(self, request_ids, group: int, width: int) -> np.ndarray:
        """The block tables of these requests, [len(request_ids), width] int32, released and unused
        entries as the null page."""
        slots = [self.requests[rid].slot for rid in request_ids]
        rows = self._rows[group]
        if width > rows.shape[1]:
            self._set_row(group, 0, width - 1, NULL_PAGE)
            rows = self._rows[group]
        return rows[slots, :width]

    def views(self, call_index: int, step) -> List[CacheView]:
        """What the layer call at `call_index` of the running order sees during `step`: one view per
        need of its block, in the block's order."""
        out = []
        for g, plane in self.where[call_index]:
            grp = self.groups[g]
            if grp.paged:
                out.append(CacheView(group=g, pages=grp.data[plane], block_table=step.block_tables[g],
                                     page_size=self.page_size))
            else:
                out.append(CacheView(group=g, state=grp.data[plane]))
        return out

    def view(self, call_index: int, step) -> CacheView:
        """The first (for most layers: the only) view of `views`, or an empty one."""
        v = self.views(call_index, step)
        return v[0] if v else CacheView()
