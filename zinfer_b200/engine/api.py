"""The Python entry point, in the reference's manner: an engine object that is
set up once from a model folder (``GeneratorRuntime.init``,
src/app/cli/runtime/generator.zig:15-46) and then generates from prompts with
per-call options (``generateFromPrompt``, generator.zig:53-123).  Token ids in,
token ids out: the reference's tokenizer and chat template are not part of this
engine, so its id-level command is the model (``generate-token-ids``,
src/app/cli/inspect.zig:246-312).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, replace
from typing import Optional, Sequence

import torch

from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, StepPlan


@dataclass
class GenerationResult:
    request_id: object
    prompt_token_ids: list[int]
    token_ids: list[int]
    finish_reason: str            # stop | length | capacity
    preemptions: int = 0


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class Engine:
    """Model, cache, scheduler and sampler on one GPU.

    ``Engine(model_dir)`` reads config.json and model.safetensors;
    ``Engine(config=cfg, random_weights_seed=s)`` draws random weights instead.
    ``kv_cache_tokens`` sizes the page pool (default: ``max_requests`` requests of
    ``max_model_len`` tokens, capped by free device memory)."""

    def __init__(self, model_dir: Optional[str] = None, *, config=None, random_weights_seed: Optional[int] = None,
                 dtype="bfloat16", device="cuda:0", page_size: int = 16, kv_cache_tokens: Optional[int] = None,
                 num_pages: Optional[int] = None, max_model_len: Optional[int] = None,
                 max_batched_tokens: int = 2048, chunk_size: Optional[int] = None, max_requests: int = 64):
        tdtype = _DTYPES.get(dtype)
        if tdtype is None:
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
        kw = dict(dtype=tdtype, device=device, max_model_len=max_model_len, page_size=page_size,
                  max_requests=max_requests)
        self._pool_args = (kv_cache_tokens, num_pages)
        sizing = self._size_pool(model_dir, config, tdtype, device, page_size, max_model_len, max_requests)
        if model_dir is not None:
            self.runner = ModelRunner.from_model_dir(model_dir, num_pages=sizing, **kw)
        elif config is not None:
            self.runner = ModelRunner.from_config(config, 0 if random_weights_seed is None else random_weights_seed,
                                                  num_pages=sizing, **kw)
        else:
            raise ValueError("give a model folder, or a configuration with random_weights_seed")
        model = self.runner.model
        self.scheduler = Scheduler(self.runner.manager, max_batched_tokens=max_batched_tokens,
                                   max_running=max_requests, chunk_size=chunk_size, max_model_len=model.max_positions)
        self.sampler = Sampler(model.spec.vocab_size, max_requests, model.device)
        self._ids = itertools.count()
        self._live: dict[object, Request] = {}

    def _size_pool(self, model_dir, config, dtype, device, page_size, max_model_len, max_requests) -> int:
        kv_cache_tokens, num_pages = self._pool_args
        if num_pages is not None:
            return num_pages
        if kv_cache_tokens is None:
            from ..config.registry import load_config
            cfg = config if config is not None else load_config(model_dir)[1]
            limit = min(getattr(cfg, "max_position_embeddings", 4096), max_model_len or 1 << 30)
            kv_cache_tokens = max_requests * min(limit, 8192)
        return max(1, -(-kv_cache_tokens // page_size))

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None, request_id=None):
        params = params or SamplingParams()
        rid = next(self._ids) if request_id is None else request_id
        V = self.runner.model.spec.vocab_size
        bad = [t for t in prompt_ids if not 0 <= int(t) < V]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the vocabulary of {V}")
        eos = tuple(params.eos_token_ids) if params.eos_token_ids is not None else self.runner.model.spec.eos_token_ids
        req = Request(rid, [int(t) for t in prompt_ids], params, eos_token_ids=eos)
        self.scheduler.add(req)
        self.sampler.begin_request(rid, params, req.prompt)
        self._live[rid] = req
        return rid

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # ---------------------------------------------------------------------- step
    def step(self) -> list[GenerationResult]:
        """One scheduler decision, one step of the model, one token for every request
        that reached its end.  Returns the requests that finished."""
        plan: StepPlan = self.scheduler.schedule()
        sampled: list[int] = []
        if plan.scheduled:
            entries, rows = [], []
            for s in plan.scheduled:
                toks = s.request.tokens[s.start:s.start + s.count]
                entries.append(StepEntry(s.request.request_id, toks, [s.count - 1] if s.samples else []))
                if s.samples:
                    rows.append(s.request)
            logits = self.runner.step(entries)
            if rows:
                tokens = self.sampler.sample(logits, [r.request_id for r in rows], [r.params for r in rows],
                                             [len(r.output) for r in rows])
                sampled = tokens.cpu().tolist()   # the step's one read back to the host
        finished = self.scheduler.update(plan, sampled)
        out = []
        for r in finished:
            self.sampler.end_request(r.request_id)
            self._live.pop(r.request_id, None)
            out.append(GenerationResult(r.request_id, r.prompt, list(r.output), r.finish_reason, r.preemptions))
        return out

    # ------------------------------------------------------------------ generate
    def generate(self, prompt_ids: Sequence[Sequence[int]], params=None, **options) -> list[GenerationResult]:
        """Generates for every prompt (lists of token ids) and returns the results in
        the prompts' order.  ``params`` is one :class:`SamplingParams` for all, or one
        per prompt; keyword options (``max_new_tokens=..., temperature=...``)
        override its fields."""
        if prompt_ids and isinstance(prompt_ids[0], int):
            prompt_ids = [prompt_ids]
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompt_ids)
        if len(params) != len(prompt_ids):
            raise ValueError("one SamplingParams per prompt, or one for all")
        if options:
            params = [replace(p, **options) for p in params]
        ids = [self.add_request(p, sp) for p, sp in zip(prompt_ids, params)]
        done: dict[object, GenerationResult] = {}
        while self.has_unfinished():
            for res in self.step():
                done[res.request_id] = res
        return [done[i] for i in ids]


def generate(model_dir: str, prompt_ids, params: Optional[SamplingParams] = None, *, dtype="bfloat16",
             engine_options: Optional[dict] = None, **options) -> list[GenerationResult]:
    """One-call form: build an :class:`Engine` for ``model_dir`` and generate."""
    return Engine(model_dir, dtype=dtype, **(engine_options or {})).generate(prompt_ids, params, **options)
