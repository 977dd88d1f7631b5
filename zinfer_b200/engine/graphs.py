"""CUDA graphs for decode steps.

A decode step (one token per request) launches some ten kernels per layer; issued
one by one from the host they cost more time than the GPU needs to run them.  For
each batch-size bucket the step is therefore captured once into a CUDA graph over
arrays of fixed address (:class:`StaticStepBuffers`) and replayed: per step the host
fills the arrays, copies them to the device once and launches the graph.  The
kernels read request lengths and block tables from those arrays, so one graph
serves every step of its bucket.  The same kernels run as in an uncaptured step.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from .batch import StaticStepBuffers, StepEntry, build_step

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


class DecodeGraphs:
    def __init__(self, runner, max_batch: int):
        self.runner = runner
        self.max_batch = max_batch
        self.width = -(-runner.model.max_positions // runner.manager.page_size)
        self._buckets: dict[int, dict] = {}
        self.replays = 0
        self.launches = 0          # kernel launches replayed through graphs so far

    def bucket_for(self, n: int) -> Optional[int]:
        for b in BUCKETS:
            if n <= b and b <= max(self.max_batch, 1):
                return b
        return n if n <= self.max_batch else None

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        return (len(entries) <= self.max_batch and all(len(e.tokens) == 1 for e in entries)
                and self.bucket_for(len(entries)) is not None)

    def run(self, entries: Sequence[StepEntry], prev_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits [bucket, vocab] (a buffer that the next replay overwrites); the
        first len(entries) rows belong to the entries, in order."""
        runner = self.runner
        b = self.bucket_for(len(entries))
        state = self._buckets.get(b)
        if state is None:
            state = self._buckets[b] = {"static": StaticStepBuffers(b, self.width, runner.device), "graph": None,
                                        "logits": None, "launches": 0, "warm": 0}
        ctx = build_step(runner.manager, entries, runner.device, runner.tile_rows, static=state["static"],
                         pf_tile_rows=runner.pf_tile_rows)
        runner.last_h2d_bytes = ctx.h2d_bytes
        if ctx.n_patch:   # outside the graph: which rows are patched changes from step to step
            ops.patch_tokens(ctx.token_ids, prev_tokens, ctx.patch_dst, ctx.patch_src)
        if state["graph"] is None:
            if state["warm"] < 1:
                # first use: run uncaptured, so that one-time set-up (function attributes,
                # rotary tables, the kernels' status word) happens outside a capture
                state["warm"] += 1
                return runner.model.forward(ctx)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.LAUNCHES
            # relaxed: a host-side call that touches no captured work (the pinned-memory allocator
            # polling an old event when Python frees a buffer) must not invalidate the capture
            with torch.cuda.graph(graph, capture_error_mode="relaxed"):
                state["logits"] = runner.model.forward(ctx)
            state["launches"] = ops.LAUNCHES - before
            ops.LAUNCHES = before
            state["graph"] = graph
        state["graph"].replay()
        self.replays += 1
        self.launches += state["launches"]
        return state["logits"]
