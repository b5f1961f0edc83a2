"""The cache manager: pages of keys and values with a block table per request, and
fixed-size state slots per request.

Calls of the run order that need keys and values of the same shape and reach (all
positions, or a window of them) form a *group*.  A group has its own pool of pages,
its own key and value tensors [calls, pages, page_size, kv_heads, head_dim] and its
own block table per request, so a windowed group can give pages back while a
full-attention group keeps them.  Calls that need a record of fixed size get a
float32 tensor [slots, *shape]; a request holds one slot id for all of them, even in
an architecture that has no such call.  A slot's records are zero when a request
receives it (`add` clears them), so no mixer ever sees its slot's previous holder.

A request's pages are given back when it ends (`free`) and, in a windowed group,
as soon as every slot of the page lies behind the window of all future queries
(`advance`).  Released block-table entries read -1; no kernel touches them because
the window bound excludes their positions.

In the reference the same duties are split between `KvStorage` (per-layer K and V
tensors [num_blocks, block_size, kv_heads, head_dim], src/kv_storage.rs:7, 92-98),
`ConvCache` (hash maps keyed by (sequence, layer), src/conv_cache.rs:33-41) and the
external scheduler crate's block tables (src/engine.rs:375-387).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..errors import CacheError
from ..parts.base import PagedNeed, StateNeed
from .pages import PagePool


@dataclass
class CacheView:
    """What one call of the run order sees of the cache."""
    kind: str                          # "paged" or "state"
    owns: bool                         # False: reads the cache another call writes
    group: int = -1                    # paged: index into StepContext.groups
    k: Optional[torch.Tensor] = None   # paged: [pages, page_size, kv_heads, head_dim]
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None   # state: float32 [slots, *shape]


@dataclass
class Group:
    need: PagedNeed
    calls: List[int]
    pool: PagePool
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None


class PageTable:
    """A request's page ids in one group, logical page -> physical page (-1 once released).
    Kept in a numpy array so that a step's batch packing copies it without conversion;
    indexing and slicing give Python ints and lists."""

    __slots__ = ("_a", "_n")

    def __init__(self):
        self._a = np.empty(16, dtype=np.int32)
        self._n = 0

    def append(self, page: int) -> None:
        if self._n == self._a.shape[0]:
            grown = np.empty(2 * self._n, dtype=np.int32)
            grown[:self._n] = self._a
            self._a = grown
        self._a[self._n] = page
        self._n += 1

    def view(self, n: Optional[int] = None) -> np.ndarray:
        return self._a[:self._n if n is None else n]

    def __len__(self) -> int:
        return self._n

    def __getitem__(self, i):
        out = self._a[:self._n][i]
        return out.tolist() if isinstance(i, slice) else int(out)

    def __setitem__(self, i: int, page: int) -> None:
        self._a[:self._n][i] = page

    def __iter__(self):
        return iter(self._a[:self._n].tolist())

    def __eq__(self, other):
        return list(self) == list(other)

    def __repr__(self):
        return f"PageTable({list(self)})"


@dataclass
class RequestCache:
    slot: int
    tokens: int = 0                              # positions covered by reserved pages
    computed: int = 0                            # positions whose keys are written
    tables: List[PageTable] = field(default_factory=list)    # per group, -1 = released
    first_live: List[int] = field(default_factory=list)     # per group: first page kept


class CacheManager:
    def __init__(self, needs: Sequence[Optional[object]], cache_of: Sequence[Optional[int]],
                 page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype = torch.float32, device="cpu", allocate: bool = True):
        """needs[i]: PagedNeed, StateNeed or None for call i of the run order;
        cache_of[i]: the call whose cache call i reads, or None.  `num_pages` pages per
        group; `max_requests` state slots.  `allocate=False` keeps only the
        bookkeeping (for tests and planning)."""
        if page_size < 1:
            raise CacheError(f"page size must be at least 1, got {page_size}")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = device
        self.groups: List[Group] = []
        self.states: Dict[int, torch.Tensor] = {}
        self.slots = PagePool(max_requests, "state slot")
        self.requests: Dict[Hashable, RequestCache] = {}
        self._views: List[Optional[CacheView]] = [None] * len(needs)
        call_group: Dict[int, int] = {}
        state_calls: Dict[tuple, List[int]] = {}
        for i, need in enumerate(needs):
            if isinstance(need, PagedNeed):
                gi = next((g for g, grp in enumerate(self.groups) if grp.need == need), None)
                if gi is None:
                    gi = len(self.groups)
                    self.groups.append(Group(need, [], PagePool(num_pages)))
                self.groups[gi].calls.append(i)
                call_group[i] = gi
            elif isinstance(need, StateNeed):
                state_calls.setdefault(tuple(need.shape), []).append(i)
                self.states[i] = None
            elif need is not None:
                raise CacheError(f"call {i}: unknown cache need {need!r}")
        # calls whose records have the same shape share one tensor [calls, slots, *shape],
        # so that a slot is cleared for all of them at once
        self._state_blocks: List[torch.Tensor] = []
        if allocate:
            for shape, calls in state_calls.items():
                block = torch.zeros((len(calls), max_requests) + shape, dtype=torch.float32,
                                    device=device)
                self._state_blocks.append(block)
                for ci, i in enumerate(calls):
                    self.states[i] = block[ci]
        for grp in self.groups:
            if allocate:
                shape = (len(grp.calls), num_pages, page_size, grp.need.num_kv_heads,
                         grp.need.head_dim)
                grp.k = torch.zeros(shape, dtype=dtype, device=device)
                grp.v = torch.zeros(shape, dtype=dtype, device=device)
        for i, need in enumerate(needs):
            src = cache_of[i] if cache_of[i] is not None else i
            owns = cache_of[i] is None
            if src in call_group:
                grp = self.groups[call_group[src]]
                ci = grp.calls.index(src)
                self._views[i] = CacheView("paged", owns, call_group[src],
                                           grp.k[ci] if allocate else None,
                                           grp.v[ci] if allocate else None)
            elif src in self.states:
                self._views[i] = CacheView("state", owns, state=self.states[src])

    # ---- what the model sees ---------------------------------------------------------

    def views(self) -> List[Optional[CacheView]]:
        return self._views

    def bytes_per_token(self) -> int:
        """Bytes of keys and values one cached token takes over all groups."""
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.calls) * g.need.num_kv_heads * g.need.head_dim * size
                   for g in self.groups)

    # ---- requests --------------------------------------------------------------------

    def has(self, req) -> bool:
        return req in self.requests

    def can_add(self) -> bool:
        return self.slots.available > 0

    def add(self, req) -> RequestCache:
        if req in self.requests:
            raise CacheError(f"request {req!r} is already live")
        rc = RequestCache(slot=self.slots.alloc(),
                          tables=[PageTable() for _ in self.groups],
                          first_live=[0 for _ in self.groups])
        # The slot's records read as zero for the new request, whoever held it before: a
        # mixer's state "before position 0" is part of this contract, not of each mixer.
        # (In stream order this comes after every step of the slot's previous holder.)
        for block in self._state_blocks:
            block[:, rc.slot].zero_()
        self.requests[req] = rc
        return rc

    def _first_needed_page(self, grp: Group, computed: int) -> int:
        """First page a query at position >= `computed` can still read."""
        if grp.need.window is None:
            return 0
        lowest_key = max(0, computed - grp.need.window + 1)
        return lowest_key // self.page_size

    def pages_needed(self, req, total_tokens: int) -> List[int]:
        """Pages each group would have to hand out to cover positions
        [0, total_tokens) of `req` (which may not be live yet)."""
        rc = self.requests.get(req)
        want = -(-total_tokens // self.page_size)
        out = []
        for gi, grp in enumerate(self.groups):
            have = len(rc.tables[gi]) if rc else 0
            out.append(max(0, want - have))
        return out

    def can_reserve(self, req, total_tokens: int) -> bool:
        return all(n <= g.pool.available
                   for n, g in zip(self.pages_needed(req, total_tokens), self.groups))

    def reserve(self, req, total_tokens: int) -> bool:
        """Hand out pages so that positions [0, total_tokens) of `req` have a slot.
        All or nothing: returns False and changes nothing when a group lacks pages."""
        rc = self.requests[req]
        if total_tokens <= rc.tokens:
            return True
        want = -(-total_tokens // self.page_size)
        if all(len(t) >= want for t in rc.tables):
            rc.tokens = total_tokens                 # room left in the last page
            return True
        if not self.can_reserve(req, total_tokens):
            return False
        for gi, grp in enumerate(self.groups):
            table = rc.tables[gi]
            while len(table) < want:
                table.append(grp.pool.alloc())
        rc.tokens = total_tokens
        return True

    def advance(self, req, computed: int) -> int:
        """Record that positions [0, computed) are written; give back the pages of
        windowed groups that no later query can see.  Returns how many were freed."""
        rc = self.requests[req]
        if computed < rc.computed:
            raise CacheError(f"request {req!r}: cannot move back from {rc.computed} "
                             f"to {computed} tokens")
        if computed > rc.tokens:
            raise CacheError(f"request {req!r}: {computed} tokens written but only "
                             f"{rc.tokens} reserved")
        rc.computed = computed
        freed = 0
        for gi, grp in enumerate(self.groups):
            first = min(self._first_needed_page(grp, computed), len(rc.tables[gi]))
            for p in range(rc.first_live[gi], first):
                grp.pool.free(rc.tables[gi][p])
                rc.tables[gi][p] = -1
                freed += 1
            rc.first_live[gi] = max(rc.first_live[gi], first)
        return freed

    def free(self, req) -> None:
        """Give back everything `req` holds."""
        rc = self.requests.pop(req, None)
        if rc is None:
            raise CacheError(f"request {req!r} is not live")
        for gi, grp in enumerate(self.groups):
            for page in rc.tables[gi]:
                if page >= 0:
                    grp.pool.free(page)
        self.slots.free(rc.slot)

    # ---- checks ----------------------------------------------------------------------

    def check(self) -> None:
        """No page lost, none held twice: every page is on the free list or in exactly
        one block table; likewise the slots."""
        for gi, grp in enumerate(self.groups):
            held = [p for rc in self.requests.values() for p in rc.tables[gi] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {gi}: a page is in two block tables")
            if len(held) != grp.pool.in_use:
                raise CacheError(f"group {gi}: {grp.pool.in_use} pages are out but block "
                                 f"tables hold {len(held)}")
            for p in held:
                if not grp.pool.is_held(p):
                    raise CacheError(f"group {gi}: page {p} is in a block table and on "
                                     f"the free list")
        slots = [rc.slot for rc in self.requests.values()]
        if len(slots) != len(set(slots)) or len(slots) != self.slots.in_use:
            raise CacheError("state slots and live requests disagree")
