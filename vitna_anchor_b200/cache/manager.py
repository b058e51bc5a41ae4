"""The cache manager: page tables on the host, pools and state arenas on the device.

A model hands over, for each of its cache layers, what that layer's mixer
needs: `KVSpec` (keys and values in pages; all of them, or a window) or
`StateSpec` (a fixed-size state per request).  Cache layers with the same
KVSpec form a group that shares page ids and has a pool of its own:

    pool[group]   [layers of the group, pages, 2 (k, v), kv heads, page_size, head_dim]
    state[cache]  [max_requests, *shape]     one row per request slot

A request holds one slot from open() to close(); its state rows are zeroed
when the slot is taken.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple, Union

import torch

from .pages import CacheError, OutOfPages, PageGroup, PageTables, UNMAPPED  # noqa: F401


@dataclass(frozen=True)
class KVSpec:
    """Keys and values of `num_kv_heads` heads of `head_dim`; window = 0 keeps every position."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """A per-request state of fixed shape, kept in the request's slot."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


CacheSpec = Union[KVSpec, StateSpec, None]


@dataclass
class LayerCacheView:
    """What one cache layer looks like to its mixer during a step."""
    spec: CacheSpec
    group: int = -1                              # page group (KVSpec)
    pages: Optional[torch.Tensor] = None         # [pages, 2, nkv, page_size, hd] of this layer
    state: Optional[torch.Tensor] = None         # [max_requests, *shape] (StateSpec)


class CacheManager:
    def __init__(self, specs: Sequence[CacheSpec], *, page_size: int, num_pages: Union[int, Sequence[int]],
                 max_requests: int, dtype: torch.dtype, device: Union[str, torch.device], allocate: bool = True):
        self.specs = list(specs)
        self.page_size = page_size
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = torch.device(device)
        by_spec: Dict[KVSpec, List[int]] = {}
        for cid, spec in enumerate(self.specs):
            if isinstance(spec, KVSpec):
                by_spec.setdefault(spec, []).append(cid)
        self.groups = [PageGroup(tuple(ids), s.num_kv_heads, s.head_dim, s.window) for s, ids in by_spec.items()]
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        self.tables = PageTables(self.groups, page_size, list(num_pages), max_requests)
        self.views: List[LayerCacheView] = [LayerCacheView(spec) for spec in self.specs]
        self.pools: List[Optional[torch.Tensor]] = []
        for g, grp in enumerate(self.groups):
            pool = None
            if allocate:
                pool = torch.zeros((len(grp.cache_ids), self.tables.pools[g].num_pages, 2, grp.num_kv_heads, page_size,
                                    grp.head_dim), dtype=dtype, device=self.device)
            self.pools.append(pool)
            for i, cid in enumerate(grp.cache_ids):
                self.views[cid].group = g
                self.views[cid].pages = pool[i] if pool is not None else None
        for cid, spec in enumerate(self.specs):
            if isinstance(spec, StateSpec) and allocate:
                self.views[cid].state = torch.zeros((max_requests, *spec.shape), dtype=spec.dtype, device=self.device)

    # -- sizes --------------------------------------------------------------------------------
    def bytes_per_token(self) -> int:
        """Cache bytes one position takes over all groups (every layer, keys and values)."""
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.cache_ids) * 2 * g.num_kv_heads * g.head_dim * size for g in self.groups)

    def token_capacity(self) -> int:
        """Positions the smallest pool can hold."""
        if not self.groups:
            return 1 << 62
        return min(p.num_pages for p in self.tables.pools) * self.page_size

    # -- requests -----------------------------------------------------------------------------
    def open(self, request_id: Hashable) -> int:
        rc = self.tables.open(request_id)
        for view in self.views:
            if view.state is not None:
                view.state[rc.slot].zero_()
        return rc.slot

    def close(self, request_id: Hashable) -> None:
        self.tables.close(request_id)

    def length(self, request_id: Hashable) -> int:
        return self.tables.get(request_id).length

    def slot(self, request_id: Hashable) -> int:
        return self.tables.get(request_id).slot

    def is_open(self, request_id: Hashable) -> bool:
        return request_id in self.tables.requests

    def reserve_step(self, plan: Sequence[Tuple[Hashable, int]]) -> None:
        """Pages for every (request, n_tokens) of a step, or OutOfPages with nothing changed."""
        if not self.tables.can_reserve(list(plan)):
            raise OutOfPages("the step needs more pages than are free")
        done = []
        try:
            for rid, n in plan:
                self.tables.reserve(rid, n)
                done.append(rid)
        except CacheError:
            for rid in done:
                self.tables.rollback(rid)
            raise

    def commit_step(self, plan: Sequence[Tuple[Hashable, int]]) -> None:
        for rid, _ in plan:
            self.tables.commit(rid)

    def rollback_step(self, plan: Sequence[Tuple[Hashable, int]]) -> None:
        for rid, _ in plan:
            self.tables.rollback(rid)

    def truncate(self, request_id: Hashable, length: int) -> None:
        """Forget positions >= length.  A fixed-size state cannot be taken back to an earlier position (it has to
        be computed again from the start), so a model with such a state refuses anything but the current length."""
        if self.has_state and length != self.length(request_id):
            raise CacheError("a request with a fixed-size state cannot be truncated; close it and run it again")
        self.tables.truncate(request_id, length)

    def rewind(self, request_id: Hashable, length: int) -> None:
        """truncate() for the step function's own undoing of steps, which restores the states itself."""
        self.tables.truncate(request_id, length)

    # -- fixed-size states across a step --------------------------------------------------------
    @property
    def has_state(self) -> bool:
        return any(v.state is not None for v in self.views)

    def save_states(self, request_ids: Sequence[Hashable]):
        """Copies of the state rows of these requests (None when no cache layer has a state): what restore_states
        needs to undo a step that wrote them."""
        if not self.has_state:
            return None
        slots = torch.tensor([self.tables.get(r).slot for r in request_ids], dtype=torch.long, device=self.device)
        return slots, [(cid, v.state.index_select(0, slots)) for cid, v in enumerate(self.views) if v.state is not None]

    def restore_states(self, saved) -> None:
        if saved is None:
            return
        slots, rows = saved
        for cid, copy in rows:
            self.views[cid].state.index_copy_(0, slots, copy)

    def free_pages(self) -> List[int]:
        return [p.free_pages for p in self.tables.pools]

    def check(self) -> None:
        self.tables.check()
