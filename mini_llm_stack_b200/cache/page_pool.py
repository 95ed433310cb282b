"""A pool of pages with a last-in-first-out free list.

Reference (serve/kv_cache.py:42,62,76): ``free_blocks = list(range(NB-1,-1,-1))``,
``pop()`` hands out page 0 first, ``free`` pushes a request's pages back in
reverse, so the page freed last is used again first.  This pool also records
the owner of every page, so that a page lost, held twice or freed twice is an
error the moment it happens.
"""

from __future__ import annotations


class PagePoolError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))
        self._owner = [None] * self.num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int, owner) -> list | None:
        """``n`` pages for ``owner``, or None (and no change) if fewer are free."""
        if n < 0:
            raise PagePoolError("cannot take a negative number of pages")
        if n > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            if self._owner[p] is not None:
                raise PagePoolError(f"page {p} was free but is owned by "
                                    f"{self._owner[p]!r}")
            self._owner[p] = owner
        self.high_water = max(self.high_water, self.num_held)
        return pages

    def give(self, pages, owner) -> None:
        """Return pages; the one given back last is handed out first."""
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise PagePoolError(f"page {p} is not in the pool")
            if self._owner[p] is None:
                raise PagePoolError(f"page {p} is freed twice")
            if self._owner[p] != owner:
                raise PagePoolError(f"page {p} belongs to {self._owner[p]!r}, "
                                    f"not to {owner!r}")
            self._owner[p] = None
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Every page is either free once or owned once."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise PagePoolError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in seen) == (self._owner[p] is not None):
                raise PagePoolError(f"page {p} is {'both free and owned' if p in seen else 'lost'}")
