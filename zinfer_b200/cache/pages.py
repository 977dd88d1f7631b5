"""A pool of equal pages (or slots) with a free list.

Pages freed last are handed out first, so reuse is immediate: a fault that comes
from stale contents of a reused page shows at once in tests.  The pool keeps the
set of pages in use and refuses to free a page that is not, so no page is ever
lost, held twice or freed twice.
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """Not enough free pages (or slots) for the request; nothing was taken."""


class PagePool:
    def __init__(self, num_pages: int, name: str = "pages"):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.name = name
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() gives 0, 1, 2, ... first
        self._used: set[int] = set()
        self._ever: set[int] = set()     # pages that have been handed out at least once
        self.reused = 0                  # allocations that returned a page which had been in use before

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return len(self._used)

    def alloc(self, n: int) -> list[int]:
        """n pages, or :class:`OutOfPages` with the pool unchanged."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"{self.name}: {n} wanted, {len(self._free)} of {self.num_pages} free")
        out = [self._free.pop() for _ in range(n)]
        self._used.update(out)
        self.reused += sum(p in self._ever for p in out)
        self._ever.update(out)
        return out

    def free(self, pages) -> None:
        pages = list(pages)
        for p in pages:
            if p not in self._used:
                raise ValueError(f"{self.name}: page {p} is not in use (freed twice, or never allocated)")
        if len(set(pages)) != len(pages):
            raise ValueError(f"{self.name}: a page is named twice in one free")
        for p in pages:
            self._used.remove(p)
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free or in use, exactly once."""
        assert len(self._free) == len(set(self._free)), "a page is on the free list twice"
        assert not (set(self._free) & self._used), "a page is both free and in use"
        assert len(self._free) + len(self._used) == self.num_pages, "a page was lost"
