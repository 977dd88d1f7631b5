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
    # For an entry of one token whose value is not yet known on the host: the row of the
    # previous step's sampled-token tensor that holds it (the token in `tokens` is a placeholder).
    token_src: Optional[int] = None


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
    tile_seq: torch.Tensor          # [tiles] request of each query tile (tiles of the exact kernel)
    tile_q0: torch.Tensor           # [tiles] first token (within the request's portion) of each query tile
    dec_seq: torch.Tensor           # [n_dec] requests that bring exactly one token
    pf_tile_seq: torch.Tensor       # [n_pf_tiles] query tiles of the tensor-core prefill kernel, over the
    pf_tile_q0: torch.Tensor        #              requests that bring more than one token
    n_dec: int
    n_pf_tiles: int
    logit_rows: Optional[torch.Tensor]   # [R] flat token indices whose logits are wanted
    kv_groups: list[KVGroupStep]
    # host copies, for parts that loop over requests
    q_lens: list[int] = field(default_factory=list)
    ctx_lens: list[int] = field(default_factory=list)   # tokens each request had in the cache before the step
    max_q_len: int = 0
    max_kv_len: int = 0
    all_decode: bool = False        # every entry brings exactly one token
    h2d_bytes: int = 0              # size of the one host->device copy that brought these arrays
    patch_dst: Optional[torch.Tensor] = None   # flat token positions to fill from the previous step's tokens
    patch_src: Optional[torch.Tensor] = None   # rows of the previous step's sampled tokens
    n_patch: int = 0


class PinnedStaging:
    """One pinned host buffer that the uncaptured steps reuse for their arrays (grown when
    a step needs more).  Reusing it keeps pinned memory from being allocated and freed
    every step; before it is overwritten, the copy of the previous step has completed."""

    def __init__(self):
        self._buf: Optional[torch.Tensor] = None
        self._copied = None

    def get(self, total: int) -> torch.Tensor:
        cuda = torch.cuda.is_available()
        if self._buf is None or self._buf.numel() < total:
            self._buf = torch.empty(max(total, 4096), dtype=torch.int32, pin_memory=cuda)
            self._copied = torch.cuda.Event() if cuda else None
        elif self._copied is not None:
            self._copied.synchronize()
        return self._buf[:total]

    def mark_copied(self) -> None:
        if self._copied is not None:
            self._copied.record()


def build_step(manager: CacheManager, entries: Sequence[StepEntry], device, tile_rows: int, pin: bool = True,
               static: Optional["StaticStepBuffers"] = None, pf_tile_rows: int = 128,
               staging: Optional[PinnedStaging] = None) -> StepContext:
    """Flattens ``entries``; their pages must already be reserved in ``manager``.

    With ``static`` (decode steps replayed from a CUDA graph) the arrays have the
    fixed capacity and addresses of those buffers: every entry brings one token, the
    batch is padded to ``static.batch`` with requests of one key in no page whose
    key/value write is skipped (slot -1), and block tables have ``static.width``
    columns."""
    n_real = len(entries)
    ps = manager.page_size
    q_lens = [len(e.tokens) for e in entries]
    ctx_lens = [manager.length(e.request_id) for e in entries]
    n_groups = len(manager.groups)
    if static is not None:
        assert all(q == 1 for q in q_lens) and n_real <= static.batch
        assert all(len(manager.block_table(e.request_id, gi)) <= static.width for e in entries for gi in range(n_groups)), \
            "a request is longer than its bucket's block tables"
        n = static.batch
        widths = [static.width] * n_groups
    else:
        n = n_real
        widths = [max(1, max(len(manager.block_table(e.request_id, gi)) for e in entries)) for gi in range(n_groups)]
    pad = n - n_real
    T = int(sum(q_lens)) + pad
    cu = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(q_lens + [1] * pad, out=cu[1:])
    n_tiles_per = [-(-q // tile_rows) for q in q_lens] + [1] * pad
    n_tiles = int(sum(n_tiles_per))
    all_q = q_lens + [1] * pad
    dec_list = [i for i, ql in enumerate(all_q) if ql == 1]
    pf_tiles = [(i, t * pf_tile_rows) for i, ql in enumerate(all_q) if ql > 1 for t in range(-(-ql // pf_tile_rows))]
    # the tiles that read the most keys come first: blocks are handed out in this order, so
    # the long ones do not end up alone at the tail
    all_ctx = ctx_lens + [0] * pad
    pf_tiles.sort(key=lambda it: -(all_ctx[it[0]] + min(all_q[it[0]], it[1] + pf_tile_rows)))
    if static is not None:
        rows = list(range(n))
    else:
        rows = [int(cu[i]) + int(w) for i, e in enumerate(entries) for w in e.want]
    R = len(rows)

    # layout of the packed buffer
    sizes = [("token_ids", T), ("positions", T), ("cu_q", n + 1), ("kv_lens", n), ("state_slots", n),
             ("tile_seq", n_tiles), ("tile_q0", n_tiles), ("logit_rows", R), ("dec_seq", len(dec_list)),
             ("pf_tile_seq", len(pf_tiles)), ("pf_tile_q0", len(pf_tiles))]
    patches = [(int(cu[i]), int(e.token_src)) for i, e in enumerate(entries) if e.token_src is not None]
    n_patch_cap = n if static is not None else len(patches)
    sizes += [("patch_dst", n_patch_cap), ("patch_src", n_patch_cap)]
    for gi in range(n_groups):
        sizes += [(f"slots{gi}", T), (f"bt{gi}", n * widths[gi])]
    offs, total = {}, 0
    for name, sz in sizes:
        offs[name] = (total, sz)
        total += -(-sz // 4) * 4   # keep every array 16-byte aligned
    if static is not None:
        host = static.host_buffer(total)
    elif staging is not None:
        host = staging.get(max(total, 4))
    else:
        host = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=pin and torch.cuda.is_available())
    buf = host.numpy()

    def arr(name):
        o, s = offs[name]
        return buf[o:o + s]

    tok, pos = arr("token_ids"), arr("positions")
    tseq, tq0 = arr("tile_seq"), arr("tile_q0")
    tok[:] = 0
    pos[:] = 0
    ti = 0
    for i in range(n):
        a, b = int(cu[i]), int(cu[i + 1])
        if i < n_real:
            tok[a:b] = np.maximum(np.asarray(entries[i].tokens, dtype=np.int64), 0)   # placeholders are patched on the device
            pos[a:b] = np.arange(ctx_lens[i], ctx_lens[i] + q_lens[i])
        for t in range(n_tiles_per[i]):
            tseq[ti] = i
            tq0[ti] = t * tile_rows
            ti += 1
    arr("cu_q")[:] = cu
    arr("dec_seq")[:] = dec_list
    if n_patch_cap:
        arr("patch_dst")[:] = -1
        arr("patch_src")[:] = 0
        arr("patch_dst")[:len(patches)] = [d for d, _ in patches]
        arr("patch_src")[:len(patches)] = [s_ for _, s_ in patches]
    arr("pf_tile_seq")[:] = [i for i, _ in pf_tiles]
    arr("pf_tile_q0")[:] = [t for _, t in pf_tiles]
    kv = arr("kv_lens")
    kv[:] = 1
    if n_real:
        kv[:n_real] = np.asarray(ctx_lens) + np.asarray(q_lens)
    ss = arr("state_slots")
    ss[:] = 0
    ss[:n_real] = [manager.requests[e.request_id].state_slot for e in entries]
    if R:
        arr("logit_rows")[:] = rows
    for gi in range(n_groups):
        W = widths[gi]
        bt = arr(f"bt{gi}").reshape(n, W)
        bt[:] = -1
        sl = arr(f"slots{gi}")
        sl[:] = -1
        for i, e in enumerate(entries):
            table = np.asarray(manager.block_table(e.request_id, gi), dtype=np.int64)
            bt[i, :len(table)] = table
            a, b = int(cu[i]), int(cu[i + 1])
            p = pos[a:b].astype(np.int64)
            pages = table[p // ps]
            if (pages < 0).any():
                raise RuntimeError(f"request {e.request_id!r}: a token would be written to a page already given back")
            sl[a:b] = pages * ps + p % ps

    if static is not None:
        dev = static.device_buffer(total)
        dev.copy_(host[:total], non_blocking=True)
        static.mark_copied()
    else:
        dev = host.to(device, non_blocking=True)
        if staging is not None:
            staging.mark_copied()

    def view(name):
        o, s = offs[name]
        return dev[o:o + s]

    groups = [KVGroupStep(view(f"slots{gi}"), view(f"bt{gi}").view(n, widths[gi])) for gi in range(n_groups)]
    return StepContext(
        n_seqs=n, n_tokens=T, token_ids=view("token_ids"), positions=view("positions"), cu_q=view("cu_q"),
        kv_lens=view("kv_lens"), state_slots=view("state_slots"), tile_seq=view("tile_seq"), tile_q0=view("tile_q0"),
        dec_seq=view("dec_seq"), pf_tile_seq=view("pf_tile_seq"), pf_tile_q0=view("pf_tile_q0"),
        n_dec=len(dec_list), n_pf_tiles=len(pf_tiles),
        patch_dst=view("patch_dst") if n_patch_cap else None, patch_src=view("patch_src") if n_patch_cap else None,
        n_patch=len(patches),
        logit_rows=view("logit_rows") if R else None, kv_groups=groups, q_lens=q_lens, ctx_lens=ctx_lens,
        max_q_len=max(q_lens, default=0),
        # a captured graph serves later steps with longer requests: its launches are shaped by the
        # bucket's length, never by the lengths of the step that happened to be captured
        max_kv_len=static.max_kv_len if static is not None else max((c + q for c, q in zip(ctx_lens, q_lens)), default=0),
        all_decode=all(q == 1 for q in q_lens), h2d_bytes=int(total) * 4)


class StaticStepBuffers:
    """Pinned host and device buffers of fixed address for the decode steps of one
    batch-size bucket, so that a captured CUDA graph finds every step's arrays at the
    same place."""

    def __init__(self, batch: int, width: int, device, max_kv_len: int = 0):
        self.batch = batch
        self.width = width                # columns of every block table
        self.max_kv_len = max_kv_len      # the longest request the bucket serves (0: unknown)
        self.device = device
        self._host = None
        self._dev = None
        self._copied = None

    def host_buffer(self, total: int) -> torch.Tensor:
        """The pinned staging buffer, safe to overwrite: the copy of the previous
        step's arrays to the device has completed."""
        if self._host is None:
            self._host = torch.zeros(total, dtype=torch.int32, pin_memory=torch.cuda.is_available())
            self._copied = torch.cuda.Event() if torch.cuda.is_available() else None
        elif self._copied is not None:
            self._copied.synchronize()
        assert self._host.numel() == total, "the layout of a bucket's arrays must not change"
        return self._host

    def mark_copied(self) -> None:
        if self._copied is not None:
            self._copied.record()

    def device_buffer(self, total: int) -> torch.Tensor:
        if self._dev is None:
            self._dev = torch.zeros(total, dtype=torch.int32, device=self.device)
        return self._dev
