"""A pool of page ids with a free list, and a pool of state slots.

Pages are handed out last-freed-first, so a page that a finished request gave back
is the next one used: reuse is the common case, not a corner.  The pool refuses a
page that is freed twice or that it never handed out.  (In the reference the pool
belongs to the external `kv-cache-scheduler` crate and is visible only as
`pool.available()` and `pool.total_allocs`, src/engine.rs:361, 629.)
"""
from __future__ import annotations

from typing import List

from ..errors import CacheError


class PagePool:
    def __init__(self, num_pages: int, what: str = "page"):
        if num_pages < 0:
            raise CacheError(f"a pool cannot have {num_pages} {what}s")
        self.num_pages = num_pages
        self.what = what
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = bytearray(num_pages)
        self.total_allocs = 0
        self.high_water = 0

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} (all {self.num_pages} in use)")
        page = self._free.pop()
        self._held[page] = 1
        self.total_allocs += 1
        self.high_water = max(self.high_water, self.in_use)
        return page

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"{self.what} {page} does not exist")
        if not self._held[page]:
            raise CacheError(f"{self.what} {page} is freed twice")
        self._held[page] = 0
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return bool(self._held[page])
