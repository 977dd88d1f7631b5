"""The cache manager: which pages and which state slot each request holds.

Keys and values live in pages of ``page_size`` tokens.  Caches with the same need
(kv heads, head size, window) form a *group*: a group has a page pool of its own
and one block table per request, valid for every cache of the group.  A request's
pages are given back when it ends, and, in a group with a window, as soon as the
window has passed them.  Beside the pages, each request holds one slot for
per-request state of fixed size (used by mixers that keep a state instead of keys;
Qwen3 has none, the slot is still allocated and freed).

This is bookkeeping on the host and touches no device; the device memory the ids
refer to is owned by :class:`zinfer_b200.cache.storage.CacheStorage`.  The
bookkeeping itself (pools, block tables, windows) is native code
(``csrc/host_runtime.cpp``), because every step of every request passes through it;
this class groups the caches, keeps the names, and is its Python face.

The reference has no counterpart: it preallocates one contiguous cache per request
(src/model/runtime/optimized_kv_cache/cache.zig:38-84) and only resets a cursor
when a slot is reused (cache.zig:109-111).
"""
from __future__ import annotations

import ctypes
import itertools
from dataclasses import dataclass
from typing import Hashable, Optional

from ..csrc import host
from .pages import GroupPool, OutOfPages


@dataclass(frozen=True)
class KVNeedKey:
    num_kv_heads: int
    head_dim: int
    window: Optional[int]


@dataclass
class KVGroup:
    key: KVNeedKey
    caches: list[str]          # names of the caches that share this group's pages
    pool: GroupPool

    @property
    def window(self) -> Optional[int]:
        return self.key.window


class RequestCache:
    """What a live request holds (read from the native manager when asked)."""

    def __init__(self, manager: "CacheManager", request_id: Hashable, native_id: int, state_slot: int):
        self._manager = manager
        self.request_id = request_id
        self.native_id = native_id
        self.state_slot = state_slot

    @property
    def length(self) -> int:
        """Tokens committed to the cache."""
        return self._manager.length(self.request_id)

    @property
    def tables(self) -> list[list[int]]:
        """Per group: page id per block, -1 once released."""
        return [self._manager.block_table(self.request_id, gi) for gi in range(len(self._manager.groups))]


class CacheManager:
    def __init__(self, kv_needs: dict[str, "KVNeedKey"], state_caches: list[str], page_size: int,
                 num_pages: int | dict[KVNeedKey, int], max_requests: int):
        """``kv_needs`` maps a cache name to what it needs; ``num_pages`` is the size
        of each group's pool (one number for all groups, or one per need)."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        keys: list[KVNeedKey] = []
        members: list[list[str]] = []
        sizes: list[int] = []
        self.group_of: dict[str, tuple[int, int]] = {}   # cache name -> (group, index within the group)
        for name, need in kv_needs.items():
            key = KVNeedKey(need.num_kv_heads, need.head_dim, need.window)
            if key.window is not None and key.window <= 0:
                raise ValueError(f"cache {name!r}: window must be positive")
            if key in keys:
                gi = keys.index(key)
                self.group_of[name] = (gi, len(members[gi]))
                members[gi].append(name)
            else:
                keys.append(key)
                members.append([name])
                sizes.append(int(num_pages[key] if isinstance(num_pages, dict) else num_pages))
                self.group_of[name] = (len(keys) - 1, 0)
        if any(n < 0 for n in sizes):
            raise ValueError("num_pages must be >= 0")
        self._lib = host.lib()
        n = len(keys)
        windows = (ctypes.c_int * max(n, 1))(*[k.window or 0 for k in keys])
        pages = (ctypes.c_int * max(n, 1))(*sizes)
        self._handle = self._lib.zi_cache_create(n, windows, pages, page_size, max_requests)
        if not self._handle:
            raise ValueError("the cache manager could not be created")
        self.groups: list[KVGroup] = [
            KVGroup(key, names, GroupPool(self._handle, gi, f"kv pages of group {gi}"))
            for gi, (key, names) in enumerate(zip(keys, members))]
        self.state_caches = list(state_caches)
        self.slots = GroupPool(self._handle, -1, "request slots")
        self.requests: dict[Hashable, RequestCache] = {}
        self._next_id = itertools.count(1)
        self._pairs = (ctypes.c_int * 4096)()      # (group, page) pairs that a call gave back
        self._info = (ctypes.c_int * 3)()
        self._per_group = (ctypes.c_int * max(n, 1))()
        # called with (group index, pages) whenever pages go back to their pool: a debugging hook
        # (the storage can overwrite what they held, so that a read of a stale page shows)
        self.on_release = None

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.zi_cache_destroy(handle)

    @property
    def handle(self):
        """The native manager (for the native step builder)."""
        return self._handle

    def native_id(self, request_id: Hashable) -> int:
        return self._live(request_id).native_id

    def _live(self, request_id: Hashable) -> RequestCache:
        rc = self.requests.get(request_id)
        if rc is None:
            raise KeyError(f"request {request_id!r} is not live (freed twice?)")
        return rc

    def _released(self, n: int) -> list[tuple[int, int]]:
        pairs = [(self._pairs[2 * i], self._pairs[2 * i + 1]) for i in range(min(n, len(self._pairs) // 2))]
        if self.on_release is not None and pairs:
            by_group: dict[int, list[int]] = {}
            for gi, page in pairs:
                by_group.setdefault(gi, []).append(page)
            for gi, pages in by_group.items():
                self.on_release(gi, pages)
        return pairs

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id: Hashable) -> RequestCache:
        if request_id in self.requests:
            raise KeyError(f"request {request_id!r} is already live")
        nid = next(self._next_id)
        slot = self._lib.zi_cache_add(self._handle, nid)
        if slot == host.OUT_OF_PAGES:
            raise OutOfPages(f"request slots: 1 wanted, 0 of {self.max_requests} free")
        if slot < 0:
            raise RuntimeError(f"adding request {request_id!r} failed (code {slot})")
        rc = RequestCache(self, request_id, nid, slot)
        self.requests[request_id] = rc
        return rc

    def has_request(self, request_id: Hashable) -> bool:
        return request_id in self.requests

    def free_request(self, request_id: Hashable) -> None:
        rc = self._live(request_id)
        if self.on_release is not None:      # the hook wants every page, however many: read the tables first
            tables = rc.tables
        n = self._lib.zi_cache_free(self._handle, rc.native_id, self._pairs, len(self._pairs))
        if n < 0:
            raise RuntimeError(f"freeing request {request_id!r} failed: {host.last_error()}")
        del self.requests[request_id]
        if self.on_release is not None:
            for gi, table in enumerate(tables):
                pages = [p for p in table if p >= 0]
                if pages:
                    self.on_release(gi, pages)

    # --------------------------------------------------------------------- pages
    def pages_needed(self, request_id: Hashable, n_new: int) -> list[int]:
        """Pages each group must still allocate so that ``n_new`` more tokens fit."""
        self._lib.zi_cache_pages_needed(self._handle, self._live(request_id).native_id, n_new, self._per_group)
        return list(self._per_group[:len(self.groups)])

    def can_reserve(self, request_id: Hashable, n_new: int) -> bool:
        return self._lib.zi_cache_can_reserve(self._handle, self._live(request_id).native_id, n_new) == 1

    def _out_of_pages(self, what: str) -> OutOfPages:
        gi, need, free = self._info[0], self._info[1], self._info[2]
        return OutOfPages(f"{what}: {need} pages wanted in {self.groups[gi].pool.name}, {free} free")

    def reserve(self, request_id: Hashable, n_new: int) -> None:
        """Pages for positions ``length .. length + n_new - 1`` in every group, or
        :class:`OutOfPages` with nothing taken."""
        rc = self._lib.zi_cache_reserve(self._handle, self._live(request_id).native_id, n_new, self._info)
        if rc == host.OUT_OF_PAGES:
            raise self._out_of_pages(f"request {request_id!r}")

    def reserve_all(self, request_ids, n_new) -> None:
        """Pages for several requests at once: all of them, or :class:`OutOfPages` with nothing taken."""
        n = len(request_ids)
        ids = (ctypes.c_longlong * max(n, 1))(*[self._live(r).native_id for r in request_ids])
        new = (ctypes.c_longlong * max(n, 1))(*[int(v) for v in n_new])
        rc = self._lib.zi_cache_reserve_all(self._handle, n, ids, new, self._info)
        if rc == host.OUT_OF_PAGES:
            raise self._out_of_pages("the step")

    def slots_for(self, request_id: Hashable, group: int, start: int, n: int) -> list[int]:
        """Flat slot (page * page_size + offset) of positions ``start .. start+n-1``."""
        out = (ctypes.c_int * max(n, 1))()
        rc = self._lib.zi_cache_slots_for(self._handle, self._live(request_id).native_id, group, start, n, out)
        if rc == host.RELEASED:
            raise RuntimeError(f"request {request_id!r}: {host.last_error()}")
        if rc < 0:
            raise IndexError(f"request {request_id!r}: {host.last_error()}")
        return list(out[:n])

    def commit(self, request_id: Hashable, n_new: int) -> list[tuple[int, int]]:
        """The step wrote ``n_new`` tokens.  Gives back the pages that every window
        has passed; returns them as (group, page)."""
        n = self._lib.zi_cache_commit(self._handle, self._live(request_id).native_id, n_new, self._pairs, len(self._pairs))
        if n < 0:
            raise RuntimeError(f"committing to request {request_id!r} failed: {host.last_error()}")
        return self._released(n) if n else []

    def length(self, request_id: Hashable) -> int:
        return int(self._lib.zi_cache_length(self._handle, self._live(request_id).native_id))

    def block_table(self, request_id: Hashable, group: int) -> list[int]:
        nid = self._live(request_id).native_id
        n = self._lib.zi_cache_table_len(self._handle, nid, group)
        if n < 0:
            raise IndexError(f"no group {group}")
        out = (ctypes.c_int * max(n, 1))()
        self._lib.zi_cache_table(self._handle, nid, group, out, n)
        return list(out[:n])

    def blocks_held(self, request_id: Hashable) -> int:
        """Blocks (pages, released ones included) that the request's shortest block table spans."""
        nid = self._live(request_id).native_id
        return min((self._lib.zi_cache_table_len(self._handle, nid, gi) for gi in range(len(self.groups))), default=0)

    # ---------------------------------------------------------------- accounting
    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    def min_free_pages(self) -> int:
        return min((g.pool.num_free for g in self.groups), default=0)

    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot either."""
        assert self._lib.zi_cache_check(self._handle) == 0, host.last_error()
        assert self._lib.zi_cache_num_requests(self._handle) == len(self.requests), "live requests differ from the native manager's"
