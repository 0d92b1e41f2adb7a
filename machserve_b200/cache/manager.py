"""The cache manager: which pages and which state slot each request holds.

Host-side bookkeeping only; the device arrays that the ids index are made by the
engine (`CacheManager.groups` says how many pages of which shape).

* Runs of layers with the same need (the same planes per token, the same window) form a GROUP.
  A group has its own pool of pages and, per request, its own block table: entry
  i is the page that holds positions [i*page_size, (i+1)*page_size), or -1.
  One page id of a group indexes every run's array of that group.
* Pages are taken when a step is about to write positions they cover
  (`reserve`), not at admission; the reference reserves a request's whole context
  at admission (crates/mach-model/src/continuous.rs:847-883 of gqf2008/machserve).
* Pages are given back when the request ends (`release`), and, in a windowed
  group, as soon as every position they cover lies before the window of the next
  query (`commit`).
* Every request also holds one slot of the fixed-size per-request state arrays
  (the reference's `gdn_state[l] : [S, ...]`, crates/mach-model/src/batched.rs:410-415),
  cleared when the request starts.  A model without such state still gets slots;
  they cost nothing.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from ..parts.base import CacheNeed, FixedState, PagedCache
from .pool import Pool, PoolError


class OutOfPages(RuntimeError):
    """A group's pool cannot cover what a step wants to write."""


@dataclass
class CacheGroup:
    index: int
    need: PagedCache
    runs: List[int]  # entries of the run order that own a cache in this group
    pool: Pool


@dataclass
class RequestCache:
    tables: List[List[int]]  # per group: logical page -> page id or -1
    state_slot: int
    num_tokens: int = 0  # positions [0, num_tokens) have been written and committed
    reserved: int = 0  # positions [0, reserved) are covered by pages (>= num_tokens)
    covered: int = 0  # positions [0, covered) need no new page in any group: the tables reach that far


class CacheManager:
    def __init__(
        self,
        needs: Sequence[CacheNeed],
        page_size: int,
        num_pages: int,
        num_state_slots: int,
        pages_per_group: Optional[Dict[int, int]] = None,
    ):
        if page_size < 1:
            raise ValueError(f"page_size {page_size}")
        self.page_size = page_size
        self.groups: List[CacheGroup] = []
        self.group_of_run: Dict[int, int] = {}
        self.state_runs: Dict[int, FixedState] = {}
        by_need: Dict[PagedCache, int] = {}
        for run, need in enumerate(needs):
            if isinstance(need, PagedCache):
                if need not in by_need:
                    n = (pages_per_group or {}).get(len(self.groups), num_pages)
                    by_need[need] = len(self.groups)
                    self.groups.append(CacheGroup(len(self.groups), need, [], Pool(n, "page")))
                g = by_need[need]
                self.groups[g].runs.append(run)
                self.group_of_run[run] = g
            elif isinstance(need, FixedState):
                self.state_runs[run] = need
            elif need is not None:
                raise TypeError(f"run {run}: unknown cache need {need!r}")
        self.slots = Pool(num_state_slots, "state slot")
        self.requests: Dict[Hashable, RequestCache] = {}
        self.fresh_slots: List[int] = []  # slots handed out since the engine last cleared them
        self.dirty: set = set()  # (request, group) whose table changed since the engine last looked

    # ------------------------------------------------------------------ requests

    def begin(self, req: Hashable) -> RequestCache:
        if req in self.requests:
            raise KeyError(f"request {req!r} already holds a cache")
        slot = self.slots.alloc()
        if slot is None:
            raise OutOfPages(f"no state slot is free ({self.slots.size} in use)")
        self.fresh_slots.append(slot)
        rc = RequestCache([[] for _ in self.groups], slot)
        self.requests[req] = rc
        return rc

    def _first_needed_page(self, group: CacheGroup, query_pos: int) -> int:
        """The first logical page a query at `query_pos` (and every later one) can still read."""
        if group.need.window is None:
            return 0
        return max(0, query_pos - group.need.window + 1) // self.page_size

    def pages_missing(self, req: Hashable, new_len: int) -> List[int]:
        """Per group, how many pages `reserve(req, new_len)` would take."""
        rc = self.requests[req]
        out = []
        for g, table in zip(self.groups, rc.tables):
            last = (new_len - 1) // self.page_size if new_len > 0 else -1
            first = self._first_needed_page(g, rc.num_tokens)
            out.append(sum(1 for i in range(first, last + 1) if i >= len(table) or table[i] < 0))
        return out

    def can_reserve(self, req: Hashable, new_len: int, spare: Optional[List[int]] = None) -> bool:
        """`spare[g]` pages of each group are left out of the count (promised to someone else)."""
        if new_len <= self.requests[req].covered:
            return True  # the common case while decoding: the last page still has room
        miss = self.pages_missing(req, new_len)
        return all(m <= g.pool.num_free - (spare[g.index] if spare else 0) for m, g in zip(miss, self.groups))

    def reserve(self, req: Hashable, new_len: int) -> None:
        """Takes the pages that positions [num_tokens, new_len) will be written to.
        Takes nothing if any group cannot cover it."""
        rc = self.requests[req]
        if new_len < rc.num_tokens:
            raise ValueError(f"request {req!r} holds {rc.num_tokens} tokens, cannot shrink to {new_len}")
        if new_len <= rc.covered:
            rc.reserved = max(rc.reserved, new_len)
            return
        miss = self.pages_missing(req, new_len)
        for m, g in zip(miss, self.groups):
            if m > g.pool.num_free:
                raise OutOfPages(
                    f"group {g.index} ({g.need}) needs {m} more pages for request {req!r}, {g.pool.num_free} are free"
                )
        for g, table in zip(self.groups, rc.tables):
            last = (new_len - 1) // self.page_size if new_len > 0 else -1
            first = self._first_needed_page(g, rc.num_tokens)
            while len(table) <= last:
                table.append(-1)
            for i in range(first, last + 1):
                if table[i] < 0:
                    table[i] = g.pool.alloc()
                    self.dirty.add((req, g.index))
        rc.reserved = max(rc.reserved, new_len)
        rc.covered = min((len(t) for t in rc.tables), default=1 << 60) * self.page_size if self.groups else 1 << 60

    def commit(self, req: Hashable, new_len: int) -> None:
        """The step that wrote up to `new_len` is done; pages that every later query's window
        has passed go back to their pool."""
        rc = self.requests[req]
        if new_len > rc.reserved:
            raise ValueError(f"request {req!r}: commit of {new_len} tokens, only {rc.reserved} are reserved")
        rc.num_tokens = max(rc.num_tokens, new_len)
        for g, table in zip(self.groups, rc.tables):
            if g.need.window is None:
                continue
            keep_from = self._first_needed_page(g, rc.num_tokens)
            for i in range(min(keep_from, len(table))):
                if table[i] >= 0:
                    g.pool.free(table[i])
                    table[i] = -1
                    self.dirty.add((req, g.index))

    def release(self, req: Hashable) -> None:
        """The request has ended (or is preempted): everything it holds goes back."""
        rc = self.requests.pop(req)
        for g, table in zip(self.groups, rc.tables):
            for p in table:
                if p >= 0:
                    g.pool.free(p)
        self.slots.free(rc.state_slot)
        if rc.state_slot in self.fresh_slots:
            self.fresh_slots.remove(rc.state_slot)
        self.dirty = {(r, g) for (r, g) in self.dirty if r != req}

    # ------------------------------------------------------------------- queries

    def block_table(self, req: Hashable, group: int) -> List[int]:
        return self.requests[req].tables[group]

    def state_slot(self, req: Hashable) -> int:
        return self.requests[req].state_slot

    def num_tokens(self, req: Hashable) -> int:
        return self.requests[req].num_tokens

    def take_fresh_slots(self) -> List[int]:
        out, self.fresh_slots = self.fresh_slots, []
        return out

    def take_dirty(self) -> set:
        """(request, group) pairs whose block table changed since the last call."""
        out, self.dirty = self.dirty, set()
        return out

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def check(self) -> None:
        """Every held page is in exactly one table, every table entry is a held page."""
        for g in self.groups:
            seen = {}
            for req, rc in self.requests.items():
                for p in rc.tables[g.index]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise PoolError(f"page {p} of group {g.index} is held by {seen[p]!r} and {req!r}")
                    if not g.pool.is_held(p):
                        raise PoolError(f"page {p} of group {g.index} is in {req!r}'s table but free in the pool")
                    seen[p] = req
            if len(seen) != g.pool.num_held:
                raise PoolError(f"group {g.index}: {g.pool.num_held} pages are held, {len(seen)} are in tables (lost pages)")
        slots = [rc.state_slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.slots.num_held:
            raise PoolError("state slots are held twice or lost")
