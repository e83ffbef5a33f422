"""A plain model of the cache's book-keeping in Python: what the native cache manager of the package must do,
call for call.  The tests drive both with the same random orders of requests and compare every answer.

Written from the reference's pool and tables (inferrs-models/src/kv_cache.rs:80-139 FIFO free list, :154-222
per-request table; inferrs/src/engine.rs:746-748 release), with groups and windows added as the package has
them.  It shares no code with the package.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

RELEASED = -1  # block-table entry of a page that was given back (a window passed it)


class CacheError(RuntimeError):
    """Misuse of the cache manager (unknown request, double free, ...)."""


class OutOfPages(CacheError):
    """Not enough free pages (or no free state slot) for what was asked; nothing was changed."""


class PagePool:
    """Page ids 0..n-1 with a FIFO free list: pages are taken from the front and given back
    to the back, as the reference's pool does (kv_cache.rs:104-139)."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free: Deque[int] = deque(range(n_pages))
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free of {self.n_pages}")
        ids = [self._free.popleft() for _ in range(n)]
        for i in ids:
            self._held[i] = True
        return ids

    def give_back(self, ids: Sequence[int]):
        for i in ids:
            if not 0 <= i < self.n_pages:
                raise CacheError(f"page id {i} is outside the pool of {self.n_pages}")
            if not self._held[i]:
                raise CacheError(f"page {i} is given back twice")
        for i in ids:
            self._held[i] = False
            self._free.append(i)

    def is_held(self, i: int) -> bool:
        return self._held[i]


@dataclass(frozen=True)
class GroupLayout:
    """What the manager needs to know of a group: which keys stay visible."""

    name: str
    window: Optional[int] = None  # None: all keys; w: a query at i sees keys j with i - w < j <= i


@dataclass
class _Request:
    slot: int
    n_tokens: int = 0                     # tokens whose keys and values are in the cache
    n_reserved: int = 0                   # tokens that pages have been taken for (>= n_tokens)
    tables: List[List[int]] = field(default_factory=list)  # per group: page number -> page id or RELEASED


class CacheManager:
    """Pages of every group and state slots for up to ``max_requests`` live requests.

    A step goes: :meth:`reserve` for every request in it (all or nothing),
    run the kernels, :meth:`commit`.  :meth:`release` ends a request.
    """

    def __init__(self, groups: Sequence[GroupLayout], page_size: int, n_pages: Sequence[int], max_requests: int):
        if page_size <= 0:
            raise CacheError(f"page_size must be positive, got {page_size}")
        if len(n_pages) != len(groups):
            raise CacheError("one page count per group is needed")
        if max_requests <= 0:
            raise CacheError(f"max_requests must be positive, got {max_requests}")
        for g in groups:
            if g.window is not None and g.window <= 0:
                raise CacheError(f"group {g.name}: window must be positive, got {g.window}")
        self.groups = list(groups)
        self.page_size = page_size
        self.pools = [PagePool(n) for n in n_pages]
        self.max_requests = max_requests
        self._free_slots: Deque[int] = deque(range(max_requests))
        self._requests: Dict[Hashable, _Request] = {}

    # ---- requests and slots -------------------------------------------------
    def has(self, rid: Hashable) -> bool:
        return rid in self._requests

    @property
    def n_live(self) -> int:
        return len(self._requests)

    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self, rid: Hashable) -> int:
        """Give the request a state slot and empty block tables; returns the slot."""
        if rid in self._requests:
            raise CacheError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise OutOfPages(f"no free state slot ({self.max_requests} requests are live)")
        slot = self._free_slots.popleft()
        self._requests[rid] = _Request(slot=slot, tables=[[] for _ in self.groups])
        return slot

    def _get(self, rid: Hashable) -> _Request:
        try:
            return self._requests[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def slot(self, rid: Hashable) -> int:
        return self._get(rid).slot

    def n_tokens(self, rid: Hashable) -> int:
        return self._get(rid).n_tokens

    def block_table(self, rid: Hashable, group: int) -> List[int]:
        return self._get(rid).tables[group]

    # ---- pages --------------------------------------------------------------
    def _pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, rid: Hashable, n_new: int) -> List[int]:
        """Pages that each group has to take so that ``n_new`` more tokens fit."""
        r = self._get(rid)
        total = self._pages_for(r.n_tokens + n_new)
        return [max(0, total - len(t)) for t in r.tables]

    def can_reserve(self, wants: Dict[Hashable, int]) -> bool:
        need = [0] * len(self.groups)
        for rid, n_new in wants.items():
            for g, n in enumerate(self.pages_needed(rid, n_new)):
                need[g] += n
        return all(need[g] <= self.pools[g].n_free for g in range(len(self.groups)))

    def fit_in_order(self, rids, n_new, free) -> int:
        """How many of the requests, taken in order, fit into ``free`` pages per group (changed in place)."""
        for i, (rid, n) in enumerate(zip(rids, n_new)):
            need = self.pages_needed(rid, n)
            if any(need[g] > free[g] for g in range(len(free))):
                return i
            for g in range(len(free)):
                free[g] -= need[g]
        return len(rids)

    def reserve(self, wants: Dict[Hashable, int]):
        """Take the pages for ``wants[rid]`` more tokens of every request named, or raise
        OutOfPages and change nothing."""
        for rid, n_new in wants.items():
            if n_new <= 0:
                raise CacheError(f"request {rid!r}: a step must bring at least one token, got {n_new}")
        if not self.can_reserve(wants):
            need = [sum(self.pages_needed(rid, n)[g] for rid, n in wants.items()) for g in range(len(self.groups))]
            raise OutOfPages("pages wanted per group " + str(need) + ", free " + str([p.n_free for p in self.pools]))
        for rid, n_new in wants.items():
            r = self._get(rid)
            for g, n in enumerate(self.pages_needed(rid, n_new)):
                r.tables[g].extend(self.pools[g].take(n))
            r.n_reserved = r.n_tokens + n_new

    def commit(self, rid: Hashable, n_new: int):
        """The step wrote ``n_new`` tokens; give back the pages that every later query's window has passed."""
        r = self._get(rid)
        if r.n_tokens + n_new > r.n_reserved:
            raise CacheError(f"request {rid!r}: commit of {n_new} tokens beyond the {r.n_reserved} reserved")
        r.n_tokens += n_new
        for g, layout in enumerate(self.groups):
            if layout.window is None:
                continue
            # the next query stands at position >= n_tokens and sees keys >= n_tokens - window + 1
            first_needed = r.n_tokens - layout.window + 1
            if first_needed <= 0:
                continue
            dead = first_needed // self.page_size  # pages 0..dead-1 hold only keys < first_needed
            gone = [p for p in r.tables[g][:dead] if p != RELEASED]
            if gone:
                self.pools[g].give_back(gone)
                for i in range(dead):
                    r.tables[g][i] = RELEASED

    def release(self, rid: Hashable):
        """The request is over: all its pages and its slot are free again."""
        r = self._get(rid)
        for g, table in enumerate(r.tables):
            self.pools[g].give_back([p for p in table if p != RELEASED])
        self._free_slots.append(r.slot)
        del self._requests[rid]

    # ---- checks -------------------------------------------------------------
    def check_invariants(self):
        """No page lost, none held by two requests, free list and tables disjoint."""
        for g, pool in enumerate(self.pools):
            seen: Dict[int, Hashable] = {}
            for rid, r in self._requests.items():
                for p in r.tables[g]:
                    if p == RELEASED:
                        continue
                    if p in seen:
                        raise CacheError(f"group {g}: page {p} is held by {seen[p]!r} and {rid!r}")
                    if not pool.is_held(p):
                        raise CacheError(f"group {g}: page {p} of {rid!r} is marked free")
                    seen[p] = rid
            free = list(pool._free)
            if len(set(free)) != len(free):
                raise CacheError(f"group {g}: a page is twice in the free list")
            if set(free) & set(seen):
                raise CacheError(f"group {g}: a held page is in the free list")
            if len(free) + len(seen) != pool.n_pages:
                raise CacheError(f"group {g}: {pool.n_pages - len(free) - len(seen)} pages are lost")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots) \
                or len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("state slots are lost or held twice")
