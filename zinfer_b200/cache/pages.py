"""A pool of equal pages (or slots) with a free list.

Pages freed last are handed out first, so reuse is immediate: a fault that comes
from stale contents of a reused page shows at once in tests.  The pool keeps track
of the pages in use and refuses to free a page that is not, so no page is ever
lost, held twice or freed twice.  The bookkeeping itself is native
(``csrc/host_runtime.cpp``); this class is its Python face.
"""
from __future__ import annotations

import ctypes

from ..csrc import host


class OutOfPages(RuntimeError):
    """Not enough free pages (or slots) for the request; nothing was taken."""


class PagePool:
    def __init__(self, num_pages: int, name: str = "pages"):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.name = name
        self._lib = host.lib()
        self._handle = self._lib.zi_pool_create(num_pages)
        self._stats_buf = (ctypes.c_longlong * 4)()

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.zi_pool_destroy(handle)

    def _stats(self):
        self._lib.zi_pool_stats(self._handle, self._stats_buf)
        return self._stats_buf

    @property
    def num_pages(self) -> int:
        return int(self._stats()[0])

    @property
    def num_free(self) -> int:
        return int(self._stats()[1])

    @property
    def num_used(self) -> int:
        return int(self._stats()[2])

    @property
    def reused(self) -> int:
        """Allocations that returned a page which had been in use before."""
        return int(self._stats()[3])

    def alloc(self, n: int) -> list[int]:
        """n pages, or :class:`OutOfPages` with the pool unchanged."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        out = (ctypes.c_int * max(n, 1))()
        rc = self._lib.zi_pool_alloc(self._handle, n, out)
        if rc == host.OUT_OF_PAGES:
            raise OutOfPages(f"{self.name}: {n} wanted, {self.num_free} of {self.num_pages} free")
        return list(out[:n])

    def free(self, pages) -> None:
        pages = [int(p) for p in pages]
        arr = (ctypes.c_int * max(len(pages), 1))(*pages)
        bad = ctypes.c_int(-1)
        rc = self._lib.zi_pool_free(self._handle, arr, len(pages), ctypes.byref(bad))
        if rc == host.BAD_PAGE:
            raise ValueError(f"{self.name}: page {bad.value} is not in use (freed twice, or never allocated)")
        if rc == host.NAMED_TWICE:
            raise ValueError(f"{self.name}: page {bad.value} is named twice in one free")

    def check(self) -> None:
        """Every page is either free or in use, exactly once."""
        assert self._lib.zi_pool_check(self._handle) == 0, f"{self.name}: {host.last_error()}"


class GroupPool:
    """Read-only face of a pool that lives inside the native cache manager (a group's pages,
    or the request slots): the manager itself allocates and frees."""

    def __init__(self, cache_handle, group: int, name: str):
        self.name = name
        self._lib = host.lib()
        self._cache = cache_handle
        self._group = group
        self._stats_buf = (ctypes.c_longlong * 4)()

    def _stats(self):
        self._lib.zi_cache_pool_stats(self._cache, self._group, self._stats_buf)
        return self._stats_buf

    num_pages = PagePool.num_pages
    num_free = PagePool.num_free
    num_used = PagePool.num_used
    reused = PagePool.reused
