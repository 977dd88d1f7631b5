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
from ..csrc import host


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


_ARRAYS = ("token_ids", "positions", "cu_q", "kv_lens", "state_slots", "tile_seq", "tile_q0", "logit_rows", "dec_seq",
           "pf_tile_seq", "pf_tile_q0", "patch_dst", "patch_src")


def build_step(manager: CacheManager, entries: Sequence[StepEntry], device, tile_rows: int, pin: bool = True,
               static: Optional["StaticStepBuffers"] = None, pf_tile_rows: int = 128,
               staging: Optional[PinnedStaging] = None) -> StepContext:
    """Flattens ``entries``; their pages must already be reserved in ``manager``.  The arrays are
    filled by the native step builder (``zi_step_build`` in csrc/host_runtime.cpp, which reads the
    block tables where the native cache manager keeps them) into one pinned buffer.

    With ``static`` (decode steps replayed from a CUDA graph) the arrays have the
    fixed capacity and addresses of those buffers: every entry brings one token, the
    batch is padded to ``static.batch`` with requests of one key in no page whose
    key/value write is skipped (slot -1), and block tables have ``static.width``
    columns."""
    lib = host.lib()
    n_e = len(entries)
    n_groups = len(manager.groups)
    q_lens = [len(e.tokens) for e in entries]
    ids = np.fromiter((manager.native_id(e.request_id) for e in entries), dtype=np.int64, count=n_e)
    ql = np.asarray(q_lens, dtype=np.int32)
    if max(q_lens, default=0) == 1:
        tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=n_e)
    else:
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
    want_counts = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=n_e)
    n_want = int(want_counts.sum())
    want = np.fromiter((int(w) for e in entries for w in e.want), dtype=np.int32, count=n_want) if n_want else np.zeros(1, np.int32)
    token_src = np.fromiter((-1 if e.token_src is None else int(e.token_src) for e in entries), dtype=np.int32, count=n_e)
    n_arrays = len(_ARRAYS) + 2 * n_groups
    layout = np.zeros(2 * n_arrays + 10 + n_groups, dtype=np.int64)

    def call(buf_ptr, capacity):
        return lib.zi_step_build(manager.handle, n_e, ids.ctypes.data, ql.ctypes.data, tokens.ctypes.data,
                                 want_counts.ctypes.data, want.ctypes.data, token_src.ctypes.data,
                                 static.batch if static is not None else 0, static.width if static is not None else 0,
                                 tile_rows, pf_tile_rows, buf_ptr, capacity, layout.ctypes.data)

    total = call(None, 0)
    if total < 0:
        raise RuntimeError(f"the step cannot be built: {host.last_error()}")
    if static is not None:
        hostbuf = static.host_buffer(total)
    elif staging is not None:
        hostbuf = staging.get(max(total, 4))
    else:
        hostbuf = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=pin and torch.cuda.is_available())
    rc = call(hostbuf.data_ptr(), hostbuf.numel())
    if rc < 0:
        raise RuntimeError(f"the step cannot be built: {host.last_error()}")
    offs = {name: (int(layout[2 * i]), int(layout[2 * i + 1])) for i, name in enumerate(_ARRAYS)}
    for gi in range(n_groups):
        for j, name in enumerate((f"slots{gi}", f"bt{gi}")):
            k = len(_ARRAYS) + 2 * gi + j
            offs[name] = (int(layout[2 * k]), int(layout[2 * k + 1]))
    tail = layout[2 * n_arrays:]
    n, T, R, n_dec, n_pf, n_patch = int(tail[1]), int(tail[2]), int(tail[3]), int(tail[4]), int(tail[5]), int(tail[7])
    widths = [int(w) for w in tail[10:10 + n_groups]]
    o, sz = offs["kv_lens"]
    kv = hostbuf[o:o + n_e].tolist()
    ctx_lens = [k - q for k, q in zip(kv, q_lens)]

    if static is not None:
        dev = static.device_buffer(total)
        dev.copy_(hostbuf[:total], non_blocking=True)
        static.mark_copied()
    else:
        dev = hostbuf[:max(total, 4)].to(device, non_blocking=True)
        if staging is not None:
            staging.mark_copied()

    def view(name):
        o, s_ = offs[name]
        return dev[o:o + s_]

    n_patch_cap = offs["patch_dst"][1]
    groups = [KVGroupStep(view(f"slots{gi}"), view(f"bt{gi}").view(n, widths[gi])) for gi in range(n_groups)]
    return StepContext(
        n_seqs=n, n_tokens=T, token_ids=view("token_ids"), positions=view("positions"), cu_q=view("cu_q"),
        kv_lens=view("kv_lens"), state_slots=view("state_slots"), tile_seq=view("tile_seq"), tile_q0=view("tile_q0"),
        dec_seq=view("dec_seq"), pf_tile_seq=view("pf_tile_seq"), pf_tile_q0=view("pf_tile_q0"),
        n_dec=n_dec, n_pf_tiles=n_pf,
        patch_dst=view("patch_dst") if n_patch_cap else None, patch_src=view("patch_src") if n_patch_cap else None,
        n_patch=n_patch,
        logit_rows=view("logit_rows") if R else None, kv_groups=groups, q_lens=q_lens, ctx_lens=ctx_lens,
        max_q_len=max(q_lens, default=0),
        # a captured graph serves later steps with longer requests: its launches are shaped by the
        # bucket's length, never by the lengths of the step that happened to be captured
        max_kv_len=static.max_kv_len if static is not None else int(tail[9]),
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
