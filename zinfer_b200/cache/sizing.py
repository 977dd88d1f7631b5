"""How many pages a byte budget buys, and what a pool costs.

One page of a group holds ``page_size`` tokens of keys and of values for every
cache of the group: ``caches * 2 * kv heads * page_size * head_dim * element size``
bytes.  Every group gets the same number of pages, so one page id across all groups
costs the sum of those.  The reference sizes one contiguous cache per request by
the same product over its layers
(src/model/runtime/optimized_kv_cache/cache.zig:423-456) and prints it with its
benchmarks (src/app/cli/tools/bench/runtime.zig:74-79).
"""
from __future__ import annotations

from typing import Optional


def group_shapes(kv_needs: dict) -> list[tuple[int, int, int]]:
    """(caches, kv heads, head size) per group, grouping equal needs like the manager does."""
    groups: dict[tuple, int] = {}
    for need in kv_needs.values():
        key = (need.num_kv_heads, need.head_dim, need.window)
        groups[key] = groups.get(key, 0) + 1
    return [(n, key[0], key[1]) for key, n in groups.items()]


def bytes_per_page(kv_needs: dict, page_size: int, element_size: int) -> int:
    """Bytes that one more page in every group costs."""
    return sum(n * 2 * heads * page_size * d * element_size for n, heads, d in group_shapes(kv_needs))


def bytes_per_token(kv_needs: dict, element_size: int) -> int:
    return bytes_per_page(kv_needs, 1, element_size)


def pages_for(kv_needs: dict, page_size: int, element_size: int, *, budget_bytes: Optional[int] = None,
              tokens: Optional[int] = None) -> int:
    """Pages per group: what ``budget_bytes`` buys (floor), at most what ``tokens`` need
    (each rounded up to whole pages); at least one."""
    per_page = bytes_per_page(kv_needs, page_size, element_size)
    pages = None
    if budget_bytes is not None and per_page > 0:
        pages = max(0, budget_bytes) // per_page
    if tokens is not None:
        want = -(-tokens // page_size)
        pages = want if pages is None else min(pages, want)
    if pages is None:
        raise ValueError("give a byte budget or a token count")
    return max(1, int(pages))
