"""The cache manager: which pages and which state slot each request holds.

Keys and values live in pages of ``page_size`` tokens.  Caches with the same need
(kv heads, head size, window) form a *group*: a group has a page pool of its own
and one block table per request, valid for every cache of the group.  A request's
pages are given back when it ends, and, in a group with a window, as soon as the
window has passed them.  Beside the pages, each request holds one slot for
per-request state of fixed size (used by mixers that keep a state instead of keys;
Qwen3 has none, the slot is still allocated and freed).

This module is bookkeeping on the host and imports no device code; the device
memory the ids refer to is owned by :class:`zinfer_b200.cache.storage.CacheStorage`.

The reference has no counterpart: it preallocates one contiguous cache per request
(src/model/runtime/optimized_kv_cache/cache.zig:38-84) and only resets a cursor
when a slot is reused (cache.zig:109-111).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Optional

from .pages import OutOfPages, PagePool


@dataclass(frozen=True)
class KVNeedKey:
    num_kv_heads: int
    head_dim: int
    window: Optional[int]


@dataclass
class KVGroup:
    key: KVNeedKey
    caches: list[str]          # names of the caches that share this group's pages
    pool: PagePool

    @property
    def window(self) -> Optional[int]:
        return self.key.window


@dataclass
class RequestCache:
    request_id: Hashable
    state_slot: int
    length: int = 0                       # tokens committed to the cache
    reserved: int = 0                     # tokens with pages reserved beyond `length`
    tables: list[list[int]] = field(default_factory=list)   # per group: page id per block, -1 once released


class CacheManager:
    def __init__(self, kv_needs: dict[str, "KVNeedKey"], state_caches: list[str], page_size: int,
                 num_pages: int | dict[KVNeedKey, int], max_requests: int):
        """``kv_needs`` maps a cache name to what it needs; ``num_pages`` is the size
        of each group's pool (one number for all groups, or one per need)."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.groups: list[KVGroup] = []
        self.group_of: dict[str, tuple[int, int]] = {}   # cache name -> (group, index within the group)
        for name, need in kv_needs.items():
            key = KVNeedKey(need.num_kv_heads, need.head_dim, need.window)
            if key.window is not None and key.window <= 0:
                raise ValueError(f"cache {name!r}: window must be positive")
            for gi, g in enumerate(self.groups):
                if g.key == key:
                    self.group_of[name] = (gi, len(g.caches))
                    g.caches.append(name)
                    break
            else:
                n = num_pages[key] if isinstance(num_pages, dict) else num_pages
                self.groups.append(KVGroup(key, [name], PagePool(n, name=f"kv pages of group {len(self.groups)}")))
                self.group_of[name] = (len(self.groups) - 1, 0)
        self.state_caches = list(state_caches)
        self.slots = PagePool(max_requests, name="request slots")
        self.requests: dict[Hashable, RequestCache] = {}
        # called with (group index, pages) whenever pages go back to their pool: a debugging hook
        # (the storage can overwrite what they held, so that a read of a stale page shows)
        self.on_release = None

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id: Hashable) -> RequestCache:
        if request_id in self.requests:
            raise KeyError(f"request {request_id!r} is already live")
        slot = self.slots.alloc(1)[0]
        rc = RequestCache(request_id, slot, tables=[[] for _ in self.groups])
        self.requests[request_id] = rc
        return rc

    def has_request(self, request_id: Hashable) -> bool:
        return request_id in self.requests

    def free_request(self, request_id: Hashable) -> None:
        rc = self.requests.pop(request_id, None)
        if rc is None:
            raise KeyError(f"request {request_id!r} is not live (freed twice?)")
        for gi, (g, table) in enumerate(zip(self.groups, rc.tables)):
            pages = [p for p in table if p >= 0]
            g.pool.free(pages)
            if self.on_release is not None and pages:
                self.on_release(gi, pages)
        self.slots.free([rc.state_slot])

    # --------------------------------------------------------------------- pages
    def _blocks_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_size)

    def pages_needed(self, request_id: Hashable, n_new: int) -> list[int]:
        """Pages each group must still allocate so that ``n_new`` more tokens fit."""
        rc = self.requests[request_id]
        want = self._blocks_for(rc.length + n_new)
        return [max(0, want - len(t)) for t in rc.tables]

    def can_reserve(self, request_id: Hashable, n_new: int) -> bool:
        return all(n <= g.pool.num_free for n, g in zip(self.pages_needed(request_id, n_new), self.groups))

    def reserve(self, request_id: Hashable, n_new: int) -> None:
        """Pages for positions ``length .. length + n_new - 1`` in every group, or
        :class:`OutOfPages` with nothing taken."""
        rc = self.requests[request_id]
        need = self.pages_needed(request_id, n_new)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"request {request_id!r}: {n} pages wanted in {g.pool.name}, {g.pool.num_free} free")
        for n, g, table in zip(need, self.groups, rc.tables):
            table.extend(g.pool.alloc(n))
        rc.reserved = max(rc.reserved, n_new)

    def slots_for(self, request_id: Hashable, group: int, start: int, n: int) -> list[int]:
        """Flat slot (page * page_size + offset) of positions ``start .. start+n-1``."""
        table = self.requests[request_id].tables[group]
        ps = self.page_size
        out = []
        for pos in range(start, start + n):
            page = table[pos // ps]
            if page < 0:
                raise RuntimeError(f"position {pos} of request {request_id!r} lies in a page already given back")
            out.append(page * ps + pos % ps)
        return out

    def commit(self, request_id: Hashable, n_new: int) -> list[tuple[int, int]]:
        """The step wrote ``n_new`` tokens.  Gives back the pages that every window
        has passed; returns them as (group, page)."""
        rc = self.requests[request_id]
        rc.length += n_new
        rc.reserved = 0
        released = []
        for gi, (g, table) in enumerate(zip(self.groups, rc.tables)):
            if g.window is None:
                continue
            # the next query sits at position `length`; it reads keys > length - window
            first_needed = rc.length - g.window + 1
            n_dead = max(0, first_needed // self.page_size)
            dead = [b for b in range(min(n_dead, len(table))) if table[b] >= 0]
            if dead:
                g.pool.free([table[b] for b in dead])
                if self.on_release is not None:
                    self.on_release(gi, [table[b] for b in dead])
                for b in dead:
                    released.append((gi, table[b]))
                    table[b] = -1
        return released

    def length(self, request_id: Hashable) -> int:
        return self.requests[request_id].length

    def block_table(self, request_id: Hashable, group: int) -> list[int]:
        return self.requests[request_id].tables[group]

    # ---------------------------------------------------------------- accounting
    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    def min_free_pages(self) -> int:
        return min((g.pool.num_free for g in self.groups), default=0)

    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot either."""
        self.slots.check()
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = [p for rc in self.requests.values() for p in rc.tables[gi] if p >= 0]
            assert len(held) == len(set(held)), f"group {gi}: a page is held by two block tables"
            assert set(held) == g.pool._used, f"group {gi}: pages in use and pages in block tables differ"
        slots = [rc.state_slot for rc in self.requests.values()]
        assert len(slots) == len(set(slots)) and set(slots) == self.slots._used, "request slots are inconsistent"
