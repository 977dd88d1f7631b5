"""CUDA graphs for decode steps.

A decode step (one token per request) launches some ten kernels per layer; issued
one by one from the host they cost more time than the GPU needs to run them.  For
each batch-size bucket the step is therefore captured once into a CUDA graph over
arrays of fixed address (:class:`StaticStepBuffers`) and replayed: per step the host
fills the arrays, copies them to the device once and launches the graph.  The
kernels read request lengths and block tables from those arrays, so one graph
serves every step of its bucket.  The same kernels run as in an uncaptured step.

A bucket is (requests, context): the context bucket is the longest live request
rounded up to the next of 256, 384, 512, 768, 1024, ... tokens.  It fixes the width
of the block tables that are filled and copied every step (so short requests of a
model with a long position limit do not pay for that limit) and the length the
decode attention's split count is chosen for (so the choice follows the requests,
not a constant).  A step whose longest request outgrows the bucket moves to the
next one, which is captured when first needed.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional, Sequence

import torch

from .. import ops
from .batch import StaticStepBuffers, StepEntry, build_step

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
MIN_CONTEXT_BUCKET = 256
MAX_GRAPHS = 32                    # captured graphs kept; the one unused longest goes first


def context_bucket(n_tokens: int, limit: int) -> int:
    """The smallest of 256, 384, 512, 768, 1024, 1536, ... that holds ``n_tokens``, at most ``limit``."""
    b = MIN_CONTEXT_BUCKET
    while b < n_tokens:
        b = b * 3 // 2 if b & (b - 1) == 0 else b * 4 // 3     # 2^k -> 3*2^(k-1) -> 2^(k+1)
    return max(1, min(b, limit))


class DecodeGraphs:
    def __init__(self, runner, max_batch: int):
        self.runner = runner
        self.max_batch = max_batch
        self._buckets: "OrderedDict[tuple[int, int], dict]" = OrderedDict()
        self._pool = None          # one memory pool for all graphs: they never run at the same time
        self.replays = 0
        self.captures = 0
        self.launches = 0          # kernel launches replayed through graphs so far

    def bucket_for(self, n: int) -> Optional[int]:
        for b in BUCKETS:
            if n <= b and b <= max(self.max_batch, 1):
                return b
        return n if n <= self.max_batch else None

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        return (len(entries) <= self.max_batch and all(len(e.tokens) == 1 for e in entries)
                and self.bucket_for(len(entries)) is not None)

    def run(self, entries: Sequence[StepEntry], prev_tokens: Optional[torch.Tensor] = None):
        """Logits [bucket, vocab] and their rows' first maxima [bucket] (buffers that the next
        replay overwrites); the first len(entries) rows belong to the entries, in order."""
        runner = self.runner
        b = self.bucket_for(len(entries))
        ps = runner.manager.page_size
        longest = max(runner.manager.length(e.request_id) for e in entries) + 1
        ctx_bucket = context_bucket(longest, -(-runner.model.max_positions // ps) * ps)
        key = (b, ctx_bucket)
        state = self._buckets.get(key)
        if state is None:
            while len(self._buckets) >= MAX_GRAPHS:
                self._buckets.popitem(last=False)
            static = StaticStepBuffers(b, -(-ctx_bucket // ps), runner.device, max_kv_len=ctx_bucket)
            state = self._buckets[key] = {"static": static, "graph": None, "outputs": None, "launches": 0, "warm": 0}
        self._buckets.move_to_end(key)
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
                return runner.model.forward(ctx, argmax=True)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.LAUNCHES
            # relaxed: a host-side call that touches no captured work (the pinned-memory allocator
            # polling an old event when Python frees a buffer) must not invalidate the capture
            if self._pool is None:
                self._pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=self._pool, capture_error_mode="relaxed"):
                state["outputs"] = runner.model.forward(ctx, argmax=True)
            self.captures += 1
            state["launches"] = ops.LAUNCHES - before
            ops.LAUNCHES = before
            state["graph"] = graph
        state["graph"].replay()
        self.replays += 1
        self.launches += state["launches"]
        return state["outputs"]
