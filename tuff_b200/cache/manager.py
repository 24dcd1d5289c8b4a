"""The cache manager: paged keys and values with a block table per request,
and slots for per-request state of fixed size.

The reference holds one sequence in one contiguous fp32 cache sized at start
(src/lfm25_engine.c:46-60) and one convolution state; this manager is what a
batch of requests needs instead.

Storages and groups.  The model says, per cache storage, what it needs
(`PagedKVNeed` or `StateNeed`, or nothing).  Paged storages with the same
(kv_heads, head_dim, window) form a *group*: one page pool, one block table per
request, and a K and a V tensor `[num_pages, kv_heads, page_size, head_dim]` per
storage (V with `v_head_dim` where a need gives one), all indexed by the group's page ids.  Groups with different needs (all
keys / a window of keys, other head shapes) have pools and tables of their own.
State storages share one slot pool: a request holds one slot number, and each
storage has a tensor `[num_slots, *shape]`.

A request's life: `open` (takes a slot, zeroes its state) -> for every step
`reserve(n)` (takes the pages that positions [held, held+n) need, in every
group; all or nothing) and, once the step ran, `commit(n)` (counts the tokens
and gives back pages that a window has passed) -> `close` (everything back).
Pages are not cleared when reused: a reader is bounded by the request's length.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import PagedKVNeed, StateNeed
from .pool import OutOfPages, PoolError, UnitPool

NO_PAGE = -1


@dataclass
class PagedStorage:
    """What an attention layer sees of the cache."""
    group: int
    page_size: int
    window: int | None
    k_pages: torch.Tensor | None = None
    v_pages: torch.Tensor | None = None


@dataclass
class StateStorage:
    """What a layer with fixed-size state sees: `state[slot]` is a request's state."""
    shape: Tuple[int, ...]
    state: torch.Tensor | None = None
    fill: float = 0.0            # what a request's state holds when the request gets its slot


@dataclass
class PagedGroup:
    need: PagedKVNeed
    pool: UnitPool
    storages: List[int] = field(default_factory=list)


@dataclass
class RequestCache:
    """One live request's holdings."""
    request_id: object
    n_tokens: int = 0                                   # tokens whose keys/state are in the cache
    tables: List[List[int]] = field(default_factory=list)   # per group: page id per block, NO_PAGE once released
    slot: int = -1
    reserved: int = 0                                   # tokens reserved beyond n_tokens for the running step
    open: bool = True
    stamp: int = 0                                      # bumped whenever a table changes
    _arrays: Dict[int, tuple] = field(default_factory=dict)   # group -> (stamp, table as int32 array)

    def table_array(self, group: int) -> np.ndarray:
        """The group's table as an int32 array, rebuilt only after the table changed (a decoding
        request takes a page once in page_size steps, and its table may hold hundreds)."""
        hit = self._arrays.get(group)
        if hit is None or hit[0] != self.stamp:
            hit = self._arrays[group] = (self.stamp, np.asarray(self.tables[group], dtype=np.int32))
        return hit[1]


class CacheManager:
    def __init__(self, needs: Sequence[object], page_size: int, max_tokens: int, max_requests: int,
                 dtype: torch.dtype = torch.bfloat16, device: str | torch.device | None = None):
        """`max_tokens`: tokens the pools can hold per group (rounded down to whole pages);
        `device=None` keeps the manager host-only (no tensors), for planning and tests."""
        if page_size < 1:
            raise ValueError("page_size must be at least 1")
        self.page_size, self.max_requests = int(page_size), int(max_requests)
        self.num_pages = int(max_tokens) // self.page_size
        self.dtype, self.device = dtype, device
        self.groups: List[PagedGroup] = []
        self.storages: List[object] = []
        self.slots = UnitPool(self.max_requests, "slot")
        self.has_state = False
        self.live: Dict[object, RequestCache] = {}
        # for tests: set `owners` to a dict and every hand-out of a page is logged there as
        # (group, page) -> [request ids in the order they held it]
        self.owners: Dict[tuple, list] | None = None
        keys: Dict[PagedKVNeed, int] = {}
        for i, need in enumerate(needs):
            if need is None:
                self.storages.append(None)
            elif isinstance(need, PagedKVNeed):
                if need not in keys:
                    keys[need] = len(self.groups)
                    self.groups.append(PagedGroup(need, UnitPool(self.num_pages, "page")))
                g = keys[need]
                self.groups[g].storages.append(i)
                st = PagedStorage(g, self.page_size, need.window)
                if device is not None:
                    shape = (self.num_pages, need.kv_heads, self.page_size, need.head_dim)
                    st.k_pages = torch.empty(shape, dtype=dtype, device=device)
                    st.v_pages = torch.empty(shape[:3] + (need.v_head_dim or need.head_dim,), dtype=dtype, device=device)
                self.storages.append(st)
            elif isinstance(need, StateNeed):
                self.has_state = True
                st = StateStorage(tuple(need.shape), fill=float(need.fill))
                if device is not None:
                    st.state = torch.full((self.max_requests,) + tuple(need.shape), float(need.fill),
                                          dtype=getattr(torch, need.dtype), device=device)
                self.storages.append(st)
            else:
                raise TypeError(f"storage {i}: unknown cache need {need!r}")

    # ---- a request's life ----------------------------------------------------
    def open(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise PoolError(f"request {request_id!r} is already open")
        slot = self.slots.take(1)[0]          # every request has a slot number, state or not
        rc = RequestCache(request_id, tables=[[] for _ in self.groups], slot=slot)
        if self.device is not None:
            for st in self.storages:
                if isinstance(st, StateStorage):
                    st.state[slot].fill_(st.fill)
        self.live[request_id] = rc
        return rc

    def can_open(self) -> bool:
        return self.slots.n_free > 0

    def pages_needed(self, rc: RequestCache, n_new: int) -> List[int]:
        """Pages each group must add so that positions [held, held+n_new) have a page."""
        end = rc.n_tokens + rc.reserved + n_new
        blocks = (end + self.page_size - 1) // self.page_size
        return [max(0, blocks - len(t)) for t in rc.tables]

    def reserve(self, rc: RequestCache, n_new: int) -> None:
        """Takes the pages for the next n_new tokens in every group, or none at all."""
        if not rc.open:
            raise PoolError(f"request {rc.request_id!r} is closed")
        need = self.pages_needed(rc, n_new)
        for g, n in zip(self.groups, need):
            if n > g.pool.n_free:
                raise OutOfPages(f"request {rc.request_id!r} needs {n} more page(s) for {n_new} token(s); "
                                 f"{g.pool.n_free} of {g.pool.n_units} free")
        for gi, (g, n, table) in enumerate(zip(self.groups, need, rc.tables)):
            if n:
                pages = g.pool.take(n)
                table.extend(pages)
                rc.stamp += 1
                if self.owners is not None:
                    for pg in pages:
                        self.owners.setdefault((gi, pg), []).append(rc.request_id)
        rc.reserved += n_new

    def cancel(self, rc: RequestCache) -> None:
        """Undoes reservations of a step that did not run."""
        blocks = (rc.n_tokens + self.page_size - 1) // self.page_size
        for g, table in zip(self.groups, rc.tables):
            while len(table) > blocks:
                g.pool.give_back(table.pop())
                rc.stamp += 1
        rc.reserved = 0

    def commit(self, rc: RequestCache, n_new: int) -> None:
        """The step ran: n_new more tokens are cached.  Gives back pages that lie wholly
        before the window of the next token."""
        if n_new > rc.reserved:
            raise PoolError(f"request {rc.request_id!r}: committing {n_new} tokens, {rc.reserved} reserved")
        rc.n_tokens += n_new
        rc.reserved -= n_new
        for g, table in zip(self.groups, rc.tables):
            w = g.need.window
            if w is None:
                continue
            first_needed = rc.n_tokens - w + 1          # oldest key the next token sees
            b = 0
            while (b + 1) * self.page_size <= first_needed and b < len(table):
                if table[b] != NO_PAGE:
                    g.pool.give_back(table[b])
                    table[b] = NO_PAGE
                    rc.stamp += 1
                b += 1

    def close(self, rc: RequestCache) -> None:
        if not rc.open:
            raise PoolError(f"request {rc.request_id!r} closed twice")
        for g, table in zip(self.groups, rc.tables):
            for p in table:
                if p != NO_PAGE:
                    g.pool.give_back(p)
            table.clear()
        rc.stamp += 1
        self.slots.give_back(rc.slot)
        rc.open = False
        rc.slot = -1
        self.live.pop(rc.request_id, None)

    # ---- views for a step ----------------------------------------------------
    def block_table(self, group: int, rcs: Sequence[RequestCache], width: int | None = None) -> np.ndarray:
        """int32 [len(rcs), width]: page id of every block of every row (NO_PAGE where none)."""
        w = max([len(rc.tables[group]) for rc in rcs] + [1]) if width is None else width
        out = np.full((len(rcs), w), NO_PAGE, dtype=np.int32)
        for i, rc in enumerate(rcs):
            t = rc.table_array(group)
            out[i, :t.size] = t
        return out

    def free_tokens(self) -> int:
        """Tokens that the scarcest group can still take."""
        if not self.groups:
            return 1 << 60
        return min(g.pool.n_free for g in self.groups) * self.page_size

    def check(self) -> None:
        """Every page is free or held by exactly one live request; same for slots."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen: Dict[int, object] = {}
            for rc in self.live.values():
                for p in rc.tables[gi]:
                    if p == NO_PAGE:
                        continue
                    if p in seen:
                        raise PoolError(f"page {p} of group {gi} held by {seen[p]!r} and {rc.request_id!r}")
                    seen[p] = rc.request_id
            if sorted(seen) != g.pool.held_units():
                raise PoolError(f"group {gi}: pages held by requests {sorted(seen)} != pages out of the pool "
                                f"{g.pool.held_units()}")
        self.slots.check()
        slots = sorted(rc.slot for rc in self.live.values())
        if slots != self.slots.held_units():
            raise PoolError(f"slots held by requests {slots} != slots out of the pool {self.slots.held_units()}")
