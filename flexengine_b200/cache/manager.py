"""The cache manager: paged keys/values per group of layers, block tables per request,
and slots for per-request state of fixed size.

The reference keeps one pool for all layers and one table per request
(src/flexengine/engine/kv_cache/allocator.py:25-67,103-127); here each cache group (all
keys, a window of keys, fixed-size state) has its own pool and its own table per
request, with a page size of its own where its spec names one, so that layers with different
needs share neither a page size nor a lifetime.
A request's pages are given back when it ends (allocator.py:103-105) or, in a window
group, once the window has passed them.  ``reserve`` is atomic across groups.

Storage of a paged group: ``[slots, 2, pages, kv_heads, page_size, head_dim]`` (keys at
index 0, values at 1), so one (page, head) tile is contiguous.
"""
from __future__ import annotations

import math
from collections import Counter
from dataclasses import dataclass, field

import numpy as np
import torch

from .page_pool import CacheExhausted, PagePool

RELEASED = -1      # block-table entry of a page that a window has passed


@dataclass
class RequestCache:
    request_id: str
    tokens: int = 0                                   # tokens whose keys/values are in the cache
    tables: list = field(default_factory=list)        # per group: list of page ids (RELEASED where given back)
    state_slot: int = -1
    room: int = 0                                     # tokens the tables have room for (the least over the paged groups)


class PagedGroup:
    def __init__(self, spec, num_pages: int, page_size: int, dtype, device, max_requests: int = 1):
        self.spec = spec
        self.page_size = int(page_size)
        self.pool = PagePool(num_pages)
        self.storage = torch.zeros((spec.slots, 2, num_pages, spec.kv_heads, self.page_size, spec.head_dim),
                                   dtype=dtype, device=device)
        # the block tables once more, as one matrix with a row per seat (a request's state slot): what a step's
        # metadata is gathered from with a few array operations instead of a loop over requests and pages
        self.table_rows = np.full((max_requests, 64), RELEASED, dtype=np.int32)

    def mirror(self, seat: int, first: int, pages) -> None:
        """Entries ``first ..`` of seat ``seat``'s table are now ``pages``."""
        need = first + len(pages)
        if need > self.table_rows.shape[1]:
            wider = np.full((self.table_rows.shape[0], max(need, 2 * self.table_rows.shape[1])), RELEASED, dtype=np.int32)
            wider[:, :self.table_rows.shape[1]] = self.table_rows
            self.table_rows = wider
        self.table_rows[seat, first:need] = pages

    def clear_row(self, seat: int, first: int = 0) -> None:
        self.table_rows[seat, first:] = RELEASED

    def kv_slot(self, slot: int):
        return self.storage[slot, 0], self.storage[slot, 1]

    def bytes_per_token(self) -> int:
        return 2 * self.spec.slots * self.spec.kv_heads * self.spec.head_dim * self.storage.element_size()


class StateGroup:
    def __init__(self, spec, max_requests: int, device):
        self.spec = spec
        dtype = getattr(torch, spec.state_dtype)
        self.storage = torch.zeros((spec.slots, max_requests) + tuple(spec.state_shape), dtype=dtype, device=device)


class CacheManager:
    def __init__(self, group_specs, num_pages, page_size: int, max_requests: int, dtype=torch.float32,
                 device="cpu"):
        """``num_pages``: pages per paged group (an int for all, or a list per group).  ``page_size``: tokens a
        page for groups whose spec names none.  An int ``num_pages`` is meant for pages of that default size: a
        group with another page size gets as many pages as hold the same number of tokens."""
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.device = torch.device(device)
        self.dtype = dtype
        self.specs = list(group_specs)
        self.groups = []
        for gi, spec in enumerate(self.specs):
            if spec.kind == "state":
                self.groups.append(StateGroup(spec, self.max_requests, self.device))
            else:
                own = int(getattr(spec, "page_size", 0) or self.page_size)
                if isinstance(num_pages, (list, tuple)):
                    n = num_pages[gi]
                else:
                    n = -(-num_pages * self.page_size // own)
                self.groups.append(PagedGroup(spec, n, own, dtype, self.device, self.max_requests))
        self.requests: dict[str, RequestCache] = {}
        self.free_state_slots = list(range(self.max_requests - 1, -1, -1))
        self._paged = [(gi, g) for gi, g in enumerate(self.groups) if isinstance(g, PagedGroup)]
        self._windowed = [(gi, g) for gi, g in self._paged if g.spec.kind == "window" and g.spec.window > 0]
        self.chunk_granularity = math.lcm(*[int(getattr(spec, "chunk_granularity", 1)) for spec in self.specs] or [1])
        # complete pages in every group: what may be shared between requests
        self.sharing_unit = math.lcm(*[g.page_size for _, g in self._paged] or [1])

    # --- sizes -----------------------------------------------------------------------------
    @property
    def paged(self):
        return self._paged

    @property
    def free_pages(self) -> int:
        return min((g.pool.free_pages for _, g in self.paged), default=0)

    @property
    def used_pages(self) -> int:
        return max((g.pool.used_pages for _, g in self.paged), default=0)

    @property
    def total_pages(self) -> int:
        return min((g.pool.num_pages for _, g in self.paged), default=0)

    def capacity_tokens(self) -> int:
        """Tokens one request could hold if it had every page."""
        return min((g.pool.num_pages * g.page_size for _, g in self.paged), default=0)

    def tokens_of(self, request_id: str) -> int:
        rc = self.requests.get(request_id)
        return rc.tokens if rc else 0

    def holds_pages(self, request_id: str) -> bool:
        rc = self.requests.get(request_id)
        return bool(rc) and any(p != RELEASED for t in rc.tables for p in t)

    # --- life cycle -------------------------------------------------------------------------
    def admit(self, request_id: str) -> RequestCache:
        """Give the request a state slot (zeroed) and empty block tables."""
        if request_id in self.requests:
            return self.requests[request_id]
        if not self.free_state_slots:
            raise CacheExhausted("no free state slot")
        slot = self.free_state_slots.pop()
        for g in self.groups:
            if isinstance(g, StateGroup) and g.storage.numel():
                g.storage[:, slot].zero_()
        rc = RequestCache(request_id, 0, [[] for _ in self.groups], slot, 0 if self._paged else 1 << 62)
        self.requests[request_id] = rc
        return rc

    def _pages_needed(self, rc: RequestCache, gi: int, target_tokens: int) -> int:
        need = -(-target_tokens // self.groups[gi].page_size)
        return max(0, need - len(rc.tables[gi]))

    def reserve(self, request_id: str, target_tokens: int) -> None:
        """Make room for the request's first ``target_tokens`` tokens in every paged group, or
        raise CacheExhausted having changed nothing."""
        if target_tokens < 0:
            raise ValueError("negative target_tokens")
        rc = self.requests.get(request_id)
        fresh = rc is None
        if fresh:
            rc = self.admit(request_id)
        elif rc.room >= target_tokens:
            return                      # already reserved (the usual case in decode)
        needs = [(gi, g, self._pages_needed(rc, gi, target_tokens)) for gi, g in self.paged]
        short = [(g.spec.name, n, g.pool.free_pages) for _, g, n in needs if n > g.pool.free_pages]
        if short:
            if fresh:
                self.free(request_id)
            name, n, have = short[0]
            raise CacheExhausted(f"Need {n} pages in group {name!r}; only {have} free")
        for gi, g, n in needs:
            if n:
                pages = g.pool.allocate(n)
                g.mirror(rc.state_slot, len(rc.tables[gi]), pages)
                rc.tables[gi].extend(pages)
        rc.room = self._room(rc)

    def _room(self, rc: RequestCache) -> int:
        return min((len(rc.tables[gi]) * g.page_size for gi, g in self._paged), default=1 << 62)

    def reserved_tokens(self, request_id: str) -> int:
        rc = self.requests.get(request_id)
        if rc is None:
            return 0
        return min((len(rc.tables[gi]) * g.page_size for gi, g in self.paged), default=1 << 62)

    def commit(self, request_id: str, count: int) -> None:
        """``count`` more tokens of the request are now in the cache; pages that a window has
        passed are given back."""
        rc = self.requests[request_id]
        target = rc.tokens + count
        for gi, g in self._paged:
            if len(rc.tables[gi]) * g.page_size < target:
                raise IndexError("KV slots not reserved")
        rc.tokens = target
        for gi, g in self._windowed:
            w = g.spec.window
            # the next query sits at position >= rc.tokens and sees keys t > position - w
            first_needed = rc.tokens - w + 1
            table = rc.tables[gi]
            for j in range(min(len(table), max(0, first_needed) // g.page_size)):
                if table[j] != RELEASED:
                    g.pool.release(table[j])
                    table[j] = RELEASED
                    g.table_rows[rc.state_slot, j] = RELEASED

    def free(self, request_id: str) -> None:
        rc = self.requests.pop(request_id, None)
        if rc is None:
            return
        for gi, g in self.paged:
            for page in rc.tables[gi]:
                if page != RELEASED:
                    g.pool.release(page)
            g.clear_row(rc.state_slot)
        self.free_state_slots.append(rc.state_slot)

    def truncate(self, request_id: str, gi: int, keep: int) -> None:
        """Give back the pages of group ``gi`` beyond the first ``keep`` (a reservation that is undone)."""
        rc = self.requests[request_id]
        g = self.groups[gi]
        for page in rc.tables[gi][keep:]:
            if page != RELEASED:
                g.pool.release(page)
        del rc.tables[gi][keep:]
        g.clear_row(rc.state_slot, keep)
        rc.room = self._room(rc)

    def share_prefix(self, donor_id: str, request_id: str, tokens: int) -> None:
        """Let a new request hold the donor's first complete pages too (reference counts,
        allocator.py:84-95); shared pages are never written again because only complete
        pages are shared and writes go to positions past them."""
        if request_id in self.requests and self.requests[request_id].tokens:
            raise ValueError("request already has cached tokens")
        donor = self.requests[donor_id]
        shared = tokens // self.sharing_unit * self.sharing_unit       # complete pages in every group
        if shared > donor.tokens:
            raise ValueError("donor has not cached that many complete pages")
        if any(g.spec.kind != "full" for _, g in self.paged):
            raise ValueError("only groups that keep every key can share a prefix")
        rc = self.admit(request_id)
        for gi, g in self.paged:
            pages = donor.tables[gi][:shared // g.page_size]
            for page in pages:
                g.pool.retain(page)
            rc.tables[gi] = list(pages)
            g.mirror(rc.state_slot, 0, rc.tables[gi])
        rc.tokens = shared
        rc.room = self._room(rc)

    # --- per-step views ------------------------------------------------------------------------
    def slot_mapping(self, request_id: str, gi: int, start: int, count: int) -> list[int]:
        """Flat slot (page * page_size + offset) of tokens start..start+count-1 in group ``gi``."""
        rc = self.requests[request_id]
        table = rc.tables[gi]
        ps = self.groups[gi].page_size
        if start < 0 or start + count > len(table) * ps:
            raise IndexError("KV slots not reserved")
        out = []
        for pos in range(start, start + count):
            page = table[pos // ps]
            if page == RELEASED:
                raise IndexError("writing to a page that was given back")
            if self.groups[gi].pool.refs[page] > 1:
                raise RuntimeError("cannot write a shared immutable KV block")
            out.append(page * ps + pos % ps)
        return out

    def table(self, request_id: str, gi: int) -> list[int]:
        return self.requests[request_id].tables[gi]

    # --- checks ---------------------------------------------------------------------------------
    def assert_invariants(self) -> None:
        for gi, g in self.paged:
            owners = Counter(p for rc in self.requests.values() for p in rc.tables[gi] if p != RELEASED)
            g.pool.assert_invariants(dict(owners))
            for rc in self.requests.values():          # the matrix of table rows says what the lists say
                row = g.table_rows[rc.state_slot]
                n = len(rc.tables[gi])
                if row[:n].tolist() != rc.tables[gi] or (row[n:] != RELEASED).any():
                    raise AssertionError(f"the table row of {rc.request_id!r} in group {g.spec.name!r} differs from its table")
            held = {rc.state_slot for rc in self.requests.values()}
            for seat in range(self.max_requests):
                if seat not in held and (g.table_rows[seat] != RELEASED).any():
                    raise AssertionError(f"seat {seat} is free but its table row is not empty")
        slots = [rc.state_slot for rc in self.requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self.free_state_slots):
            raise AssertionError("a state slot is held twice")
        if len(slots) + len(self.free_state_slots) != self.max_requests:
            raise AssertionError("a state slot was lost")
