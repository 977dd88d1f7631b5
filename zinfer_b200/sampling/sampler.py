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
        # Rows of token counts, [rows, V], made when first needed.  A request that ended in the step in
        # flight keeps its row until the host has read that step, while the requests admitted in its
        # place already hold theirs: twice the running requests is the most that can be held.
        self._counts: Optional[torch.Tensor] = None
        self._rows = PagePool(2 * max_requests, name="token-count rows")
        self._row_of: dict[Hashable, int] = {}

    # ------------------------------------------------------------ token counts
    def has_request(self, request_id: Hashable) -> bool:
        return request_id in self._row_of

    def begin_request(self, request_id: Hashable, params: SamplingParams, prompt: Sequence[int]) -> None:
        """Call once when a request is admitted (not when it is queued: a row of counts is
        [vocabulary] wide and there are only ``max_requests`` of them).  With penalties on, its
        prompt is counted as history (src/app/cli/runtime/generator.zig:95-97).  The row is kept
        until :meth:`end_request`, across preemption, so the counts of generated tokens survive."""
        if not params.has_penalties or request_id in self._row_of:
            return
        if self._counts is None:
            self._counts = torch.zeros((self._rows.num_pages, self.vocab), dtype=torch.int32, device=self.device)
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
    _FIELDS = ("temperature", "top_p", "min_p", "rep", "pres", "freq", "top_k", "draw_index", "count_rows")

    def _staging(self):
        """A flat pinned buffer of 32-bit words from a small ring (so a buffer is not overwritten
        while its copy to the device may still be in flight): for R rows its first 2 R words hold the
        seeds (64-bit each), the next len(_FIELDS) * R the per-row fields, field by field."""
        if not hasattr(self, "_ring"):
            pin = torch.cuda.is_available() and self.device.type == "cuda"
            self._ring = [torch.zeros(((2 + len(self._FIELDS)) * self.max_requests,), dtype=torch.int32, pin_memory=pin)
                          for _ in range(4)]
            self._turn = 0
        buf = self._ring[self._turn % len(self._ring)]
        self._turn += 1
        return buf

    @staticmethod
    def all_greedy(params: Sequence[SamplingParams]) -> bool:
        """Whether these rows need nothing but their logits' first maximum."""
        return all(p.greedy and not p.has_penalties for p in params)

    def sample(self, logits: torch.Tensor, request_ids: Sequence[Hashable], params: Sequence[SamplingParams],
               draw_index: Sequence[int], greedy_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token (int32, on the device) per row of ``logits``.  ``greedy_ids``: the rows' first
        maxima where the model's step has already found them."""
        R = logits.shape[0]
        assert R == len(request_ids) == len(params) == len(draw_index)
        if self.all_greedy(params):
            return greedy_ids if greedy_ids is not None else ops.argmax(logits)
        any_pen = any(p.has_penalties for p in params)
        # all per-row parameters travel in one pinned buffer and one contiguous copy; the tensors the
        # kernel takes are views of that copy
        nf = len(self._FIELDS)
        words = self._staging()[:(2 + nf) * R]
        seeds_h = words[:2 * R].view(torch.int64)
        host = words[2 * R:].view(nf, R)
        f = host.view(torch.float32)
        for i, (rid, p) in enumerate(zip(request_ids, params)):
            seeds_h[i] = p.seed
            f[0, i] = 0.0 if p.greedy else p.temperature
            f[1, i] = p.top_p
            f[2, i] = p.min_p
            f[3, i] = p.repetition_penalty
            f[4, i] = p.presence_penalty
            f[5, i] = p.frequency_penalty
            host[6, i] = p.top_k
            host[7, i] = int(draw_index[i])
            host[8, i] = self._row_of.get(rid, -1) if p.has_penalties else -1
        dev_words = words.to(self.device, non_blocking=True) if self.device.type == "cuda" else words.clone()
        seeds = dev_words[:2 * R].view(torch.int64)
        dev = dev_words[2 * R:].view(nf, R)
        fl = dev.view(torch.float32)
        return ops.sample(
            logits, temperature=fl[0], seeds=seeds, draw_index=dev[7], top_k=dev[6], top_p=fl[1], min_p=fl[2],
            repetition_penalty=fl[3] if any_pen else None, presence_penalty=fl[4] if any_pen else None,
            frequency_penalty=fl[5] if any_pen else None, count_rows=dev[8] if any_pen else None,
            counts=self._counts if any_pen else None)
