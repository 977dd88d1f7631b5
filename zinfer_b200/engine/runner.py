"""The step function: runs a batch of (request, next tokens) from the cache.

:class:`ModelRunner` owns the model, the cache manager and the device storage.
``step(entries)`` reserves pages for the tokens it is given, runs only those
tokens as one batch against what earlier steps left in the cache, commits them,
and returns the 32-bit logits at the wanted places.  Generation (the scheduler)
and trace replay both drive this one function.

The reference's unit of work is one token of one request
(src/model/runtime/optimized_decoder/runtime.zig:103-148); its prefill is a loop
over that (runtime.zig:150-163).
"""
from __future__ import annotations

from typing import Hashable, Optional, Sequence

import torch

from .. import ops, profiling
from ..cache import CacheManager, CacheStorage, OutOfPages, pages_for
from ..config.registry import load_config
from ..weights import load_tensors, random_tensors
from .batch import PinnedStaging, StepEntry, build_step
from .model import DecoderModel


class StepError(ValueError):
    """The step's input cannot be run: bad token id, too long a request, unknown request."""


def _require_cuda(device: torch.device) -> None:
    if not torch.cuda.is_available() or device.type != "cuda":
        raise RuntimeError("zinfer_b200 runs on a CUDA device only; there is no CPU path")


class ModelRunner:
    def __init__(self, model: DecoderModel, page_size: int = 16, num_pages: Optional[int] = None,
                 max_tokens: Optional[int] = None, max_requests: int = 64, cuda_graphs: bool = True,
                 kv_cache_bytes: Optional[int] = None, gpu_memory_fraction: Optional[float] = None,
                 workspace_bytes: int = 0, poison_freed_pages: bool = False):
        """The page pool is sized, in this order of precedence, by ``num_pages`` (pages per
        group), by ``kv_cache_bytes`` (a byte budget for all groups together), by
        ``gpu_memory_fraction`` (that share of the device memory which is free now, the weights
        being loaded already, minus ``workspace_bytes`` kept for activations), each capped by
        ``max_tokens`` cached tokens when that is given too; or by ``max_tokens`` alone.
        ``poison_freed_pages`` (debugging) overwrites every page with huge values when it is
        given back, so that a kernel which reads a stale page cannot go unnoticed."""
        _require_cuda(model.device)
        ops.lib()  # fail now, and loudly, if the kernel library cannot be built or loaded
        self.model = model
        self.device = model.device
        kv_needs, state_needs = model.cache_needs()
        if num_pages is None:
            elt = torch.empty((), dtype=model.dtype).element_size()
            budget = kv_cache_bytes
            if budget is None and gpu_memory_fraction is not None and model.device.type == "cuda":
                free, _total = torch.cuda.mem_get_info(model.device)
                budget = int(free * gpu_memory_fraction) - workspace_bytes
            if budget is None and max_tokens is None:
                raise ValueError("give num_pages, kv_cache_bytes, gpu_memory_fraction or max_tokens")
            num_pages = pages_for(kv_needs, page_size, elt, budget_bytes=budget, tokens=max_tokens)
        self.manager = CacheManager(kv_needs, list(state_needs), page_size, num_pages, max_requests)
        self.storage = CacheStorage(self.manager, state_needs, model.dtype, self.device)
        if poison_freed_pages:
            self.manager.on_release = self.storage.poison
        model.attach(self.storage)
        self.tile_rows = ops.attention_tile_rows()
        self.pf_tile_rows = ops.attention_prefill_tile_rows()
        self.steps_run = 0
        self.last_h2d_bytes = 0
        self._staging = PinnedStaging()
        # decode steps are replayed from CUDA graphs when every mixer can be captured
        self.graphs = None
        if cuda_graphs and model.device.type == "cuda" and all(
                getattr(b.mixer, "graph_safe", False) for b in model.blocks):
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(self, max_requests)

    # ------------------------------------------------------------- construction
    @classmethod
    def from_model_dir(cls, model_dir: str, dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                       max_model_len: Optional[int] = None, **kw) -> "ModelRunner":
        family, config = load_config(model_dir)
        model = DecoderModel(family.model_spec(config), dtype, device, max_positions=max_model_len)
        model.bind(load_tensors(model_dir, model.tensor_specs(), dtype, model.device))
        runner = cls(model, **kw)
        runner.config = config
        return runner

    @classmethod
    def from_config(cls, config, seed: int, dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                    max_model_len: Optional[int] = None, **kw) -> "ModelRunner":
        """Random weights drawn on the device (no model folder)."""
        from ..config.registry import family_for

        family = family_for(config.to_dict())
        model = DecoderModel(family.model_spec(config), dtype, device, max_positions=max_model_len)
        model.bind(random_tensors(model.tensor_specs(), seed, dtype, model.device))
        runner = cls(model, **kw)
        runner.config = config
        return runner

    @property
    def graph_launches(self) -> int:
        return self.graphs.launches if self.graphs is not None else 0

    # ------------------------------------------------------------------ requests
    def has_request(self, request_id: Hashable) -> bool:
        return self.manager.has_request(request_id)

    def add_request(self, request_id: Hashable) -> None:
        rc = self.manager.add_request(request_id)
        if self.storage.state:
            self.storage.reset_slot(rc.state_slot)

    def end_request(self, request_id: Hashable) -> None:
        """Gives back everything the request holds."""
        self.manager.free_request(request_id)

    def length(self, request_id: Hashable) -> int:
        return self.manager.length(request_id)

    # ---------------------------------------------------------------------- step
    def validate(self, entries: Sequence[StepEntry]) -> None:
        V = self.model.spec.vocab_size
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            if e.token_src is not None:
                if len(e.tokens) != 1:
                    raise StepError(f"request {e.request_id!r}: only a single token can come from the step before")
                bad = []
            else:
                bad = [t for t in e.tokens if not 0 <= int(t) < V]
            if bad:
                raise StepError(f"request {e.request_id!r}: token id {bad[0]} is outside the vocabulary of {V}")
            have = self.manager.length(e.request_id) if self.manager.has_request(e.request_id) else 0
            if have + len(e.tokens) > self.model.max_positions:
                raise StepError(f"request {e.request_id!r} would reach {have + len(e.tokens)} tokens; "
                                f"the limit is {self.model.max_positions}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is outside its {len(e.tokens)} tokens")

    def reserve(self, entries: Sequence[StepEntry]) -> None:
        """Pages for all entries, or :class:`OutOfPages` with nothing kept."""
        added = []
        try:
            for e in entries:
                if not self.manager.has_request(e.request_id):
                    self.add_request(e.request_id)
                    added.append(e.request_id)
            self.manager.reserve_all([e.request_id for e in entries], [len(e.tokens) for e in entries])
        except OutOfPages:
            for rid in added:
                self.manager.free_request(rid)
            raise

    def step(self, entries: Sequence[StepEntry], prev_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the entries as one batch; returns logits [wanted, vocab] in the order
        of the entries and of each entry's ``want`` (None if nothing is wanted).
        ``prev_tokens`` (int32, on the device) is read by entries with ``token_src``."""
        return self._step(entries, prev_tokens, False)[0]

    def step_argmax(self, entries: Sequence[StepEntry], prev_tokens: Optional[torch.Tensor] = None):
        """As :meth:`step`, and beside the logits the first maximum of every wanted row (int32, on
        the device): greedy decoding without a second pass over the logits."""
        return self._step(entries, prev_tokens, True)

    def _step(self, entries: Sequence[StepEntry], prev_tokens: Optional[torch.Tensor], argmax: bool):
        if not entries:
            return None, None
        self.validate(entries)
        if any(e.token_src is not None for e in entries) and prev_tokens is None:
            raise StepError("an entry takes its token from the step before, but no such tokens were given")
        self.reserve(entries)
        if profiling.ACTIVE is not None:
            profiling.ACTIVE.begin_step()    # profiled steps launch their kernels one by one, never from a graph
        if self.graphs is not None and profiling.ACTIVE is None and self.graphs.eligible(entries):
            all_rows, all_ids = self.graphs.run(entries, prev_tokens)
            wanted = [i for i, e in enumerate(entries) if len(e.want)]
            if not wanted:
                logits = ids = None
            elif len(wanted) == len(entries):
                logits, ids = all_rows[:len(entries)], all_ids[:len(entries)]
            else:
                pick = torch.tensor(wanted, device=self.device)
                logits, ids = all_rows[pick], (all_ids[pick] if argmax else None)
        else:
            ctx = build_step(self.manager, entries, self.device, self.tile_rows, pf_tile_rows=self.pf_tile_rows,
                             staging=self._staging)
            self.last_h2d_bytes = ctx.h2d_bytes
            if ctx.n_patch:
                ops.patch_tokens(ctx.token_ids, prev_tokens, ctx.patch_dst, ctx.patch_src)
            if argmax:
                logits, ids = self.model.forward(ctx, argmax=True)
            else:
                logits, ids = self.model.forward(ctx), None
        for e in entries:
            self.manager.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        return logits, ids
