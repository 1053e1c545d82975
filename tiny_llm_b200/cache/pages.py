"""Page pool: fixed-size pages handed out from a LIFO free list.

The reference's pool (tiny_llm/runtime/page_pool.cpp:6-61) also keeps a LIFO list whose ids come
out 0, 1, 2, ... at first, throws when more pages are asked for than are free, and finds a double
free by a linear search.  Here `allocate` returns None when the pool cannot serve the request (the
scheduler decides what happens then), and ownership is tracked per page so that a page freed
twice, or freed by a request that does not hold it, raises at once."""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional


class PageError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() gives 0, 1, 2, ...
        self._owner: Dict[int, Hashable] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, n: int, owner: Hashable) -> Optional[List[int]]:
        if n < 0:
            raise ValueError("negative page count")
        if n > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._owner[p] = owner
        return pages

    def free(self, pages: List[int], owner: Hashable) -> None:
        for p in pages:
            held_by = self._owner.get(p, None)
            if p not in self._owner:
                raise PageError(f"page {p} is freed twice (or was never handed out)")
            if held_by != owner:
                raise PageError(f"page {p} is held by {held_by!r}, not by {owner!r}")
        for p in pages:
            del self._owner[p]
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner.get(page)

    def check(self) -> None:
        """Every page is either free or owned, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageError("a page is on the free list twice")
        if free & set(self._owner):
            raise PageError("a page is both free and owned")
        if len(free) + len(self._owner) != self.num_pages:
            raise PageError("a page is lost: neither free nor owned")
