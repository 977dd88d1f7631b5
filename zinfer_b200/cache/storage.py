"""Device memory behind the cache manager's ids.

For each group one tensor ``[caches, 2, pages, kv heads, page_size, head_dim]``
(keys at index 0, values at index 1) in the run's dtype: a page id is valid for
every cache of the group.  For each state cache one tensor
``[request slots + 1, *shape]``, zeroed for a slot when a request takes it.  The last
slot belongs to no request: the rows that pad a captured decode batch name it, so a
mixer that updates ``state[state_slots]`` with device operations alone harms nobody.
"""
from __future__ import annotations

from dataclasses import dataclass
import torch

from .manager import CacheManager


@dataclass
class KVCacheView:
    """What an attention-like mixer gets for one run of its layer."""

    k: torch.Tensor          # [pages, kv heads, page_size, head_dim]
    v: torch.Tensor
    group: int               # index into StepContext.kv_groups
    page_size: int
    writes: bool             # False: this run only reads a cache another run wrote


@dataclass
class StateView:
    """What a mixer with fixed-size state gets: ``state[slot]`` belongs to the
    request whose slot is ``slot`` (StepContext.state_slots)."""

    state: torch.Tensor      # [request slots + 1, *shape]; the last slot is the padding rows' scratch
    writes: bool = True


class CacheStorage:
    def __init__(self, manager: CacheManager, state_needs: dict, dtype: torch.dtype, device):
        self.manager = manager
        self.kv: list[torch.Tensor] = []
        for g in manager.groups:
            shape = (len(g.caches), 2, g.pool.num_pages, g.key.num_kv_heads, manager.page_size, g.key.head_dim)
            self.kv.append(torch.zeros(shape, dtype=dtype, device=device))
        self.state: dict[str, torch.Tensor] = {
            name: torch.zeros((manager.max_requests + 1, *need.shape), dtype=need.dtype, device=device)
            for name, need in state_needs.items()
        }

    def kv_view(self, cache_name: str, writes: bool) -> KVCacheView:
        gi, ci = self.manager.group_of[cache_name]
        t = self.kv[gi]
        return KVCacheView(k=t[ci, 0], v=t[ci, 1], group=gi, page_size=self.manager.page_size, writes=writes)

    def state_view(self, cache_name: str, writes: bool = True) -> StateView:
        return StateView(self.state[cache_name], writes)

    def reset_slot(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()

    def poison(self, group: int, pages, value: float = 3.0e4) -> None:
        """Overwrites the keys of ``pages`` with ``value`` and their values with ``-value`` in every
        cache of the group (debugging: what a freed page held must never reach a result)."""
        idx = torch.as_tensor(list(pages), dtype=torch.long, device=self.kv[group].device)
        self.kv[group][:, 0].index_fill_(1, idx, value)
        self.kv[group][:, 1].index_fill_(1, idx, -value)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * t.element_size() for t in self.state.values())
