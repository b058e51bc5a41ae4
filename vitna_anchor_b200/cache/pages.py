"""Pages, block tables and state slots: the host side of the cache manager.

Nothing here touches a device.  A page is `page_size` consecutive positions of
one request in every layer of one group; a block table maps a request's block
number (position // page_size) to a page id, or -1 where no page is held
(before the first, or behind a window).  Pages are handed out from a LIFO
stack, so a page that was just given back is the next one used.

The reference keeps a contiguous cache per sequence slot
(engine/include/model.h:106-110) and so never runs out in mid-request; its
unused kv_cache.c names the vocabulary only (block, block table, unmapped =
all-ones).  The paging here is this engine's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional

UNMAPPED = -1


class CacheError(RuntimeError):
    """A misuse of the cache manager: a page freed twice, a foreign page, an unknown request."""


class OutOfPages(CacheError):
    """The pool cannot give the pages a step needs; nothing was changed."""


class PagePool:
    """`num_pages` page ids with an owner tag each.  alloc/free are O(1)."""

    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise CacheError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() gives 0 first
        self._owner: List[Optional[Hashable]] = [None] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def alloc(self, owner: Hashable) -> int:
        if owner is None:
            raise CacheError("a page needs an owner")
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        self._owner[page] = owner
        return page

    def free(self, page: int, owner: Hashable) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page {page} is not in the pool")
        if self._owner[page] is None:
            raise CacheError(f"page {page} is freed twice")
        if self._owner[page] != owner:
            raise CacheError(f"page {page} belongs to {self._owner[page]!r}, not to {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def owner(self, page: int) -> Optional[Hashable]:
        return self._owner[page]

    def check(self) -> None:
        """Every page is either free exactly once or owned; raises otherwise."""
        seen = set()
        for p in self._free:
            if p in seen:
                raise CacheError(f"page {p} is on the free list twice")
            if self._owner[p] is not None:
                raise CacheError(f"page {p} is free and owned")
            seen.add(p)
        owned = sum(1 for o in self._owner if o is not None)
        if owned + len(seen) != self.num_pages:
            raise CacheError("a page is lost: neither free nor owned")


class SlotPool:
    """Fixed-size per-request state slots 0..n-1; the lowest free slot is given first."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._owner: List[Optional[Hashable]] = [None] * num_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def acquire(self, owner: Hashable) -> int:
        if not self._free:
            raise CacheError("no free request slot")
        s = self._free.pop()
        self._owner[s] = owner
        return s

    def release(self, slot: int, owner: Hashable) -> None:
        if self._owner[slot] != owner or owner is None:
            raise CacheError(f"slot {slot} is not held by {owner!r}")
        self._owner[slot] = None
        self._free.append(slot)
        self._free.sort(reverse=True)


@dataclass
class GroupTable:
    """One request's pages in one layer group."""
    blocks: List[int] = field(default_factory=list)   # block number -> page id or UNMAPPED
    first_held: int = 0                               # blocks below this were given back (window)


@dataclass
class RequestCache:
    request_id: Hashable
    slot: int
    length: int = 0                # positions whose keys and values are in the cache (committed)
    reserved: int = 0              # positions reserved beyond `length` for the step in flight
    tables: Dict[int, GroupTable] = field(default_factory=dict)   # group index -> table


@dataclass(frozen=True)
class PageGroup:
    """Layers with the same needs share page ids: `window` = 0 keeps every key, else the last `window`."""
    cache_ids: tuple          # the cache layers of this group, in pool order
    num_kv_heads: int
    head_dim: int
    window: int = 0


class PageTables:
    """Requests, their block tables in every group, and the pools behind them."""

    def __init__(self, groups: List[PageGroup], page_size: int, pages_per_group: List[int], max_requests: int):
        if page_size < 1:
            raise CacheError("page_size must be at least 1")
        if len(groups) != len(pages_per_group):
            raise CacheError("one page count is needed for each group")
        self.groups = list(groups)
        self.page_size = page_size
        self.pools = [PagePool(n) for n in pages_per_group]
        self.slots = SlotPool(max_requests)
        self.requests: Dict[Hashable, RequestCache] = {}

    # -- requests ---------------------------------------------------------------------------
    def open(self, request_id: Hashable) -> RequestCache:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already open")
        rc = RequestCache(request_id, self.slots.acquire(request_id))
        rc.tables = {g: GroupTable() for g in range(len(self.groups))}
        self.requests[request_id] = rc
        return rc

    def get(self, request_id: Hashable) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not open") from None

    def close(self, request_id: Hashable) -> None:
        """Give back every page and the slot."""
        rc = self.get(request_id)
        for g, table in rc.tables.items():
            for page in table.blocks:
                if page != UNMAPPED:
                    self.pools[g].free(page, request_id)
        self.slots.release(rc.slot, request_id)
        del self.requests[request_id]

    # -- pages ------------------------------------------------------------------------------
    def _first_needed_block(self, g: int, first_query_pos: int) -> int:
        w = self.groups[g].window
        if w <= 0:
            return 0
        return max(0, first_query_pos - w + 1) // self.page_size

    def pages_needed(self, request_id: Hashable, n_tokens: int) -> List[int]:
        """New pages each group must give for the request's next n_tokens positions."""
        rc = self.get(request_id)
        end = rc.length + rc.reserved + n_tokens
        need = []
        for g in range(len(self.groups)):
            have = len(rc.tables[g].blocks)
            need.append(max(0, -(-end // self.page_size) - have))
        return need

    def can_reserve(self, plan: List[tuple]) -> bool:
        """Whether the pools hold enough for every (request_id, n_tokens) of a step together."""
        total = [0] * len(self.groups)
        for request_id, n in plan:
            for g, k in enumerate(self.pages_needed(request_id, n)):
                total[g] += k
        return all(total[g] <= self.pools[g].free_pages for g in range(len(self.groups)))

    def reserve(self, request_id: Hashable, n_tokens: int) -> None:
        """Hold pages for positions [length, length + n_tokens).  All groups or nothing."""
        rc = self.get(request_id)
        if n_tokens < 1:
            raise CacheError("a step needs at least one token of a request")
        need = self.pages_needed(request_id, n_tokens)
        for g, k in enumerate(need):
            if k > self.pools[g].free_pages:
                raise OutOfPages(f"group {g} needs {k} pages for request {request_id!r} and has {self.pools[g].free_pages} free")
        for g, k in enumerate(need):
            for _ in range(k):
                rc.tables[g].blocks.append(self.pools[g].alloc(request_id))
        rc.reserved += n_tokens

    def commit(self, request_id: Hashable) -> None:
        """The step ran: the reserved positions are now cached.  Pages a window has passed go back."""
        rc = self.get(request_id)
        rc.length += rc.reserved
        rc.reserved = 0
        for g in range(len(self.groups)):
            table = rc.tables[g]
            first = min(self._first_needed_block(g, rc.length), len(table.blocks))
            for b in range(table.first_held, first):
                if table.blocks[b] != UNMAPPED:
                    self.pools[g].free(table.blocks[b], request_id)
                    table.blocks[b] = UNMAPPED
            table.first_held = max(table.first_held, first)

    def rollback(self, request_id: Hashable) -> None:
        """The step did not run: give back the pages that only the reserved positions needed."""
        rc = self.get(request_id)
        rc.reserved = 0
        self._trim(rc, rc.length)

    def truncate(self, request_id: Hashable, length: int) -> None:
        """Forget positions >= length (cf. vitna_llama_truncate, engine/src/model.c:467-469).  A group
        with a window cannot go back behind what it has already given away."""
        rc = self.get(request_id)
        if rc.reserved:
            raise CacheError("truncate during a step")
        if length < 0 or length > rc.length:
            raise CacheError(f"cannot truncate request {request_id!r} of length {rc.length} to {length}")
        for g in range(len(self.groups)):
            if self._first_needed_block(g, length) < rc.tables[g].first_held:
                raise CacheError(f"group {g} has already given back pages that position {length} needs")
        rc.length = length
        self._trim(rc, length)

    def _trim(self, rc: RequestCache, length: int) -> None:
        keep = -(-length // self.page_size)
        for g, table in rc.tables.items():
            while len(table.blocks) > keep:
                page = table.blocks.pop()
                if page != UNMAPPED:
                    self.pools[g].free(page, rc.request_id)
            table.first_held = min(table.first_held, len(table.blocks))

    # -- what a step needs --------------------------------------------------------------------
    def slot_of_position(self, request_id: Hashable, g: int, pos: int) -> int:
        page = self.get(request_id).tables[g].blocks[pos // self.page_size]
        if page == UNMAPPED:
            raise CacheError(f"position {pos} of request {request_id!r} has no page in group {g}")
        return page * self.page_size + pos % self.page_size

    def check(self) -> None:
        """Pool consistency, and every held page is in exactly one table."""
        for g, pool in enumerate(self.pools):
            pool.check()
            held = {}
            for rc in self.requests.values():
                for page in rc.tables[g].blocks:
                    if page == UNMAPPED:
                        continue
                    if page in held:
                        raise CacheError(f"page {page} of group {g} is held by {held[page]!r} and {rc.request_id!r}")
                    if pool.owner(page) != rc.request_id:
                        raise CacheError(f"page {page} of group {g} is in a table but owned by {pool.owner(page)!r}")
                    held[page] = rc.request_id
            if len(held) + pool.free_pages != pool.num_pages:
                raise CacheError(f"group {g}: {pool.num_pages - pool.free_pages - len(held)} pages are owned but in no table")
