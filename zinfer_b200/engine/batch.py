"""The batch of one step, flattened for the kernels.

A step holds entries (request, its next tokens, the places whose logits are
wanted): portions of prompts beside single decoded tokens, cut anywhere.  All
tokens of all entries lie in one flat list; per-request arrays say where each
request's tokens start, how many keys it has, and where its pages are.  The host
fills one int32 buffer and sends it to the device in a single copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()        # indices into `tokens` whose logits are returned


@dataclass
class KVGroupStep:
    slot_mapping: torch.Tensor      # [T] page * page_size + offset, where each token's k and v go
    block_tables: torch.Tensor      # [n, W] page ids per request, -1 where none


@dataclass
class StepContext:
    n_seqs: int
    n_tokens: int
    token_ids: torch.Tensor         # [T] int32
    positions: torch.Tensor         # [T] int32, position of each token in its request
    cu_q: torch.Tensor              # [n+1] int32, first token of each request in the flat list
    kv_lens: torch.Tensor           # [n] int32, keys per request including this step's tokens
    state_slots: torch.Tensor       # [n] int32, the request's slot in the per-request state
    tile_seq: torch.Tensor          # [tiles] request of each query tile
    tile_q0: torch.Tensor           # [tiles] first token (within the request's portion) of each query tile
    logit_rows: Optional[torch.Tensor]   # [R] flat token indices whose logits are wanted
    kv_groups: list[KVGroupStep]
    # host copies, for parts that loop over requests
    q_lens: list[int] = field(default_factory=list)
    ctx_lens: list[int] = field(default_factory=list)   # tokens each request had in the cache before the step
    max_q_len: int = 0
    max_kv_len: int = 0
    all_decode: bool = False        # every entry brings exactly one token
    h2d_bytes: int = 0              # size of the one host->device copy that brought these arrays


def build_step(manager: CacheManager, entries: Sequence[StepEntry], device, tile_rows: int,
               pin: bool = True) -> StepContext:
    """Flattens ``entries``; their pages must already be reserved in ``manager``."""
    n = len(entries)
    ps = manager.page_size
    q_lens = [len(e.tokens) for e in entries]
    ctx_lens = [manager.length(e.request_id) for e in entries]
    T = int(sum(q_lens))
    cu = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(q_lens, out=cu[1:])
    n_tiles_per = [-(-q // tile_rows) for q in q_lens]
    n_tiles = int(sum(n_tiles_per))
    rows = [int(cu[i]) + int(w) for i, e in enumerate(entries) for w in e.want]
    R = len(rows)
    n_groups = len(manager.groups)
    widths = []
    for gi in range(n_groups):
        widths.append(max(1, max(len(manager.block_table(e.request_id, gi)) for e in entries)))

    # layout of the packed buffer
    sizes = [("token_ids", T), ("positions", T), ("cu_q", n + 1), ("kv_lens", n), ("state_slots", n),
             ("tile_seq", n_tiles), ("tile_q0", n_tiles), ("logit_rows", R)]
    for gi in range(n_groups):
        sizes += [(f"slots{gi}", T), (f"bt{gi}", n * widths[gi])]
    offs, total = {}, 0
    for name, sz in sizes:
        offs[name] = (total, sz)
        total += -(-sz // 4) * 4   # keep every array 16-byte aligned
    host = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=pin and torch.cuda.is_available())
    buf = host.numpy()

    def arr(name):
        o, s = offs[name]
        return buf[o:o + s]

    tok, pos = arr("token_ids"), arr("positions")
    tseq, tq0 = arr("tile_seq"), arr("tile_q0")
    ti = 0
    for i, e in enumerate(entries):
        a, b = int(cu[i]), int(cu[i + 1])
        tok[a:b] = np.asarray(e.tokens, dtype=np.int64)
        pos[a:b] = np.arange(ctx_lens[i], ctx_lens[i] + q_lens[i])
        for t in range(n_tiles_per[i]):
            tseq[ti] = i
            tq0[ti] = t * tile_rows
            ti += 1
    arr("cu_q")[:] = cu
    arr("kv_lens")[:] = np.asarray(ctx_lens) + np.asarray(q_lens) if n else 0
    arr("state_slots")[:] = [manager.requests[e.request_id].state_slot for e in entries]
    if R:
        arr("logit_rows")[:] = rows
    for gi in range(n_groups):
        W = widths[gi]
        bt = arr(f"bt{gi}").reshape(n, W)
        bt[:] = -1
        sl = arr(f"slots{gi}")
        for i, e in enumerate(entries):
            table = np.asarray(manager.block_table(e.request_id, gi), dtype=np.int64)
            bt[i, :len(table)] = table
            a, b = int(cu[i]), int(cu[i + 1])
            p = pos[a:b].astype(np.int64)
            pages = table[p // ps]
            if (pages < 0).any():
                raise RuntimeError(f"request {e.request_id!r}: a token would be written to a page already given back")
            sl[a:b] = pages * ps + p % ps

    dev = host.to(device, non_blocking=True)

    def view(name):
        o, s = offs[name]
        return dev[o:o + s]

    groups = [KVGroupStep(view(f"slots{gi}"), view(f"bt{gi}").view(n, widths[gi])) for gi in range(n_groups)]
    return StepContext(
        n_seqs=n, n_tokens=T, token_ids=view("token_ids"), positions=view("positions"), cu_q=view("cu_q"),
        kv_lens=view("kv_lens"), state_slots=view("state_slots"), tile_seq=view("tile_seq"), tile_q0=view("tile_q0"),
        logit_rows=view("logit_rows") if R else None, kv_groups=groups, q_lens=q_lens, ctx_lens=ctx_lens,
        max_q_len=max(q_lens, default=0), max_kv_len=max((c + q for c, q in zip(ctx_lens, q_lens)), default=0),
        all_decode=all(q == 1 for q in q_lens), h2d_bytes=int(host.numel()) * 4)
