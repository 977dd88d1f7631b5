"""Turns logits into one token per request on the device.

Greedy rows use the argmax kernel; the others the sampling kernel, which applies
the reference's chain in its order: penalties, top-k, temperature, min-p, top-p,
draw (src/sampling/sampler.zig:18-91).  The i-th draw of a request is a function
of its seed and i alone, so a request's tokens do not depend on what else is in
the batch nor on whether it was preempted and recomputed.
"""
from __future__ import annotations

from typing import Hashable, Optional, Sequence

import torch

from .. import ops
from ..cache.pages import PagePool
from .params import SamplingParams


class Sampler:
    def __init__(self, vocab_size: int, max_requests: int, device):
        self.vocab = vocab_size
        self.device = torch.device(device)
        self.max_requests = max_requests
        self._counts: Optional[torch.Tensor] = None      # [max_requests, V], made when first needed
        self._rows = PagePool(max_requests, name="token-count rows")
        self._row_of: dict[Hashable, int] = {}

    # ------------------------------------------------------------ token counts
    def begin_request(self, request_id: Hashable, params: SamplingParams, prompt: Sequence[int]) -> None:
        """Call once when a request enters.  With penalties on, its prompt is counted
        as history (src/app/cli/runtime/generator.zig:95-97)."""
        if not params.has_penalties:
            return
        if self._counts is None:
            self._counts = torch.zeros((self.max_requests, self.vocab), dtype=torch.int32, device=self.device)
        row = self._rows.alloc(1)[0]
        self._row_of[request_id] = row
        self._counts[row].zero_()
        if len(prompt):
            toks = torch.tensor(list(prompt), dtype=torch.int32, device=self.device)
            ops.count_tokens(self._counts[row], toks)

    def end_request(self, request_id: Hashable) -> None:
        row = self._row_of.pop(request_id, None)
        if row is not None:
            self._rows.free([row])

    # ----------------------------------------------------------------- sampling
    def sample(self, logits: torch.Tensor, request_ids: Sequence[Hashable], params: Sequence[SamplingParams],
               draw_index: Sequence[int]) -> torch.Tensor:
        """One token (int32, on the device) per row of ``logits``."""
        R = logits.shape[0]
        assert R == len(request_ids) == len(params) == len(draw_index)
        if all(p.greedy and not p.has_penalties for p in params):
            return ops.argmax(logits)
        f32 = lambda vals: torch.tensor(vals, dtype=torch.float32, device=self.device)
        i32 = lambda vals: torch.tensor(vals, dtype=torch.int32, device=self.device)
        any_pen = any(p.has_penalties for p in params)
        count_rows = i32([self._row_of.get(rid, -1) if p.has_penalties else -1 for rid, p in zip(request_ids, params)])
        return ops.sample(
            logits,
            temperature=f32([0.0 if p.greedy else p.temperature for p in params]),
            seeds=torch.tensor([p.seed for p in params], dtype=torch.int64, device=self.device),
            draw_index=i32(list(draw_index)),
            top_k=i32([p.top_k for p in params]),
            top_p=f32([p.top_p for p in params]),
            min_p=f32([p.min_p for p in params]),
            repetition_penalty=f32([p.repetition_penalty for p in params]) if any_pen else None,
            presence_penalty=f32([p.presence_penalty for p in params]) if any_pen else None,
            frequency_penalty=f32([p.frequency_penalty for p in params]) if any_pen else None,
            count_rows=count_rows if any_pen else None,
            counts=self._counts if any_pen else None)
