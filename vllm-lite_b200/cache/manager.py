"""The cache manager: pages and block tables for keys and values, slots for
per-request state of fixed size.

Entries of the running order whose needs are equal form a group.  A paged group
has one pool of pages; a request holds, per paged group, a block table whose
entry i covers positions [i * page_size, (i + 1) * page_size)
(crates/core/src/types/sequence.rs:21 and
crates/model/src/components/attention/paged_gqa.rs:50-52 of the reference).  One
page id addresses the same page in every entry of its group.  Pages are taken
when a step is about to write them (`append`), given back when the request ends
(`free`) or when a group's window has passed them (`release_behind_window`),
and used again.  A state slot is taken at admission and zeroed; fixed-state
groups index their tensors by it.

This file is bookkeeping on the host; `CacheStorage` holds the device tensors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .pool import Pool, PoolError
from .spec import FixedState, PagedKV


@dataclass
class CacheLayout:
    """Groups of entries of the running order, and for every entry where its cache lies."""
    paged_groups: List[PagedKV]
    paged_members: List[List[int]]          # order indices that own a cache in the group
    state_groups: List[FixedState]
    state_members: List[List[int]]
    call_place: List[Optional[tuple]]       # per order entry: ("paged"|"state", group, index in group, owns)

    @classmethod
    def from_needs(cls, needs: list, cache_of: list) -> "CacheLayout":
        pg, pm, sg, sm = [], [], [], []
        place: List[Optional[tuple]] = [None] * len(needs)
        for i, need in enumerate(needs):
            if cache_of[i] is not None:
                continue
            if need is None:
                continue
            if isinstance(need, PagedKV):
                groups, members, kind = pg, pm, "paged"
            elif isinstance(need, FixedState):
                groups, members, kind = sg, sm, "state"
            else:
                raise TypeError(f"order[{i}] asks for {need!r}; a cache need is PagedKV, FixedState or None")
            if need in groups:
                g = groups.index(need)
            else:
                groups.append(need)
                members.append([])
                g = len(groups) - 1
            members[g].append(i)
            place[i] = (kind, g, len(members[g]) - 1, True)
        for i, src in enumerate(cache_of):
            if src is not None:
                if place[src] is None:
                    raise ValueError(f"order[{i}] reads the cache of order[{src}], which keeps none")
                kind, g, idx, _ = place[src]
                place[i] = (kind, g, idx, False)
        return cls(pg, pm, sg, sm, place)


@dataclass
class RequestCache:
    request_id: object
    state_slot: int
    num_tokens: int = 0
    block_tables: List[List[int]] = field(default_factory=list)   # per paged group; -1 = given back


class OutOfPages(RuntimeError):
    pass


class CacheManager:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages, max_requests: int):
        """`num_pages`: one number for every paged group, or a list with one number per group."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.layout = layout
        self.page_size = int(page_size)
        n_groups = len(layout.paged_groups)
        counts = [int(num_pages)] * n_groups if isinstance(num_pages, int) else [int(n) for n in num_pages]
        if len(counts) != n_groups:
            raise ValueError(f"{n_groups} paged groups need {n_groups} page counts, got {len(counts)}")
        self.pools = [Pool(n, "page") for n in counts]
        self.slots = Pool(max_requests, "state slot")
        self.requests: Dict[object, RequestCache] = {}
        self.fresh_slots: List[int] = []      # slots handed out since the storage last zeroed them

    # ---- admission and release -------------------------------------------
    def admit(self, request_id) -> RequestCache:
        if request_id in self.requests:
            raise KeyError(f"request {request_id!r} already holds a cache")
        got = self.slots.allocate(1)
        if got is None:
            raise OutOfPages("no state slot is free")
        rc = RequestCache(request_id, got[0], 0, [[] for _ in self.pools])
        self.requests[request_id] = rc
        self.fresh_slots.append(got[0])
        return rc

    def free(self, request_id):
        rc = self.requests.pop(request_id)
        for pool, table in zip(self.pools, rc.block_tables):
            pool.release([p for p in table if p >= 0])
        self.slots.release([rc.state_slot])
        if rc.state_slot in self.fresh_slots:
            self.fresh_slots.remove(rc.state_slot)

    # ---- growth -----------------------------------------------------------
    def pages_needed(self, request_id, count: int) -> List[int]:
        """Pages each group must still take before `count` more tokens fit."""
        rc = self.requests[request_id]
        total = rc.num_tokens + count
        want = -(-total // self.page_size)
        return [max(0, want - len(t)) for t in rc.block_tables]

    def can_append(self, request_id, count: int) -> bool:
        return all(n <= pool.free_count for n, pool in zip(self.pages_needed(request_id, count), self.pools))

    def append(self, request_id, count: int) -> int:
        """Take the pages that `count` more tokens need, in every group or in none.
        Returns the position of the first new token."""
        if count <= 0:
            raise ValueError("a step brings at least one token per request")
        rc = self.requests[request_id]
        need = self.pages_needed(request_id, count)
        if any(n > pool.free_count for n, pool in zip(need, self.pools)):
            raise OutOfPages(f"request {request_id!r} needs {need} pages, free: {[p.free_count for p in self.pools]}")
        for n, pool, table in zip(need, self.pools, rc.block_tables):
            table.extend(pool.allocate(n))
        start = rc.num_tokens
        rc.num_tokens += count
        return start

    def slot_of(self, request_id, group: int, position: int) -> int:
        """page * page_size + offset of a position, for the kernels that write the cache."""
        page = self.requests[request_id].block_tables[group][position // self.page_size]
        if page < 0:
            raise PoolError(f"position {position} of request {request_id!r} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    def release_behind_window(self, request_id) -> int:
        """Give back the pages that no later query of the request can read.  The next query
        sits at position num_tokens and reads from num_tokens - window + 1 on."""
        rc = self.requests[request_id]
        freed = 0
        for need, pool, table in zip(self.layout.paged_groups, self.pools, rc.block_tables):
            if need.window is None:
                continue
            first_needed = rc.num_tokens - need.window + 1
            dead_blocks = min(max(first_needed, 0) // self.page_size, len(table))
            gone = [table[b] for b in range(dead_blocks) if table[b] >= 0]
            for b in range(dead_blocks):
                table[b] = -1
            pool.release(gone)
            freed += len(gone)
        return freed

    def take_fresh_slots(self) -> List[int]:
        out, self.fresh_slots = self.fresh_slots, []
        return out

    # ---- figures and checks -------------------------------------------------
    def free_pages(self) -> List[int]:
        return [p.free_count for p in self.pools]

    def check_invariants(self):
        """No page lost, none held twice, none both free and held."""
        for g, pool in enumerate(self.pools):
            pool.check()
            seen = {}
            for rc in self.requests.values():
                for p in rc.block_tables[g]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise PoolError(f"page {p} of group {g} is held by {seen[p]!r} and {rc.request_id!r}")
                    if not pool.is_held(p):
                        raise PoolError(f"page {p} of group {g} is in a block table but free")
                    seen[p] = rc.request_id
            if len(seen) != pool.held_count:
                raise PoolError(f"group {g}: {pool.held_count} pages are held but block tables name {len(seen)}")
        self.slots.check()
        slots = [rc.state_slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.slots.held_count:
            raise PoolError("state slots and requests disagree")
