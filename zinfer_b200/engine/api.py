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

from .. import ops, profiling
from ..sampling import Sampler, SamplingParams, analyze_generated
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, StepPlan


@dataclass
class _InFlight:
    """A launched step whose sampled tokens the host has not read yet."""

    plan: StepPlan
    tokens_dev: Optional[torch.Tensor]     # [rows] int32 on the device
    tokens_host: Optional[torch.Tensor]    # the pinned copy (valid once `done` has completed)
    done: Optional[object]
    row_of: dict                           # request id -> row of tokens_dev


@dataclass
class GenerationResult:
    request_id: object
    prompt_token_ids: list[int]
    token_ids: list[int]
    finish_reason: str            # stop | length | capacity | abort
    preemptions: int = 0


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class Engine:
    """Model, cache, scheduler and sampler on one GPU.

    ``Engine(model_dir)`` reads config.json and the safetensors file(s);
    ``Engine(config=cfg, random_weights_seed=s)`` draws random weights instead.

    The page pool is sized by the first of these that is given: ``num_pages`` (pages per
    cache group), ``kv_cache_tokens`` (cached tokens), ``kv_cache_bytes`` (a byte budget for
    keys and values of all layers).  With none of them the pool takes ``gpu_memory_fraction``
    of the device memory that is free once the weights are loaded, less what a step's
    activations need, but never more than ``max_requests`` requests of ``max_model_len``
    tokens could fill.  (The reference sizes one cache per request for prompt + max_new_tokens,
    src/app/cli/runtime/generator.zig:70-79; its byte count is
    src/model/runtime/optimized_kv_cache/cache.zig:423-456.)"""

    def __init__(self, model_dir: Optional[str] = None, *, config=None, random_weights_seed: Optional[int] = None,
                 dtype="bfloat16", device="cuda:0", page_size: int = 16, kv_cache_tokens: Optional[int] = None,
                 num_pages: Optional[int] = None, kv_cache_bytes: Optional[int] = None,
                 gpu_memory_fraction: float = 0.9, max_model_len: Optional[int] = None,
                 max_batched_tokens: int = 2048, chunk_size: Optional[int] = None, max_requests: int = 64,
                 pipelined: bool = True):
        tdtype = _DTYPES.get(dtype)
        if tdtype is None:
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
        if not 0.0 < gpu_memory_fraction <= 1.0:
            raise ValueError("gpu_memory_fraction must lie in (0, 1]")
        if model_dir is not None:
            from ..config.registry import load_config
            cfg = load_config(model_dir)[1]
        elif config is not None:
            cfg = config
        else:
            raise ValueError("give a model folder, or a configuration with random_weights_seed")
        kw = dict(dtype=tdtype, device=device, max_model_len=max_model_len, page_size=page_size,
                  max_requests=max_requests)
        if num_pages is not None:
            kw["num_pages"] = num_pages
        elif kv_cache_tokens is not None:
            kw["max_tokens"] = kv_cache_tokens
        else:
            limit = min(getattr(cfg, "max_position_embeddings", 4096), max_model_len or 1 << 30)
            per_request = -(-limit // page_size) * page_size
            if kv_cache_bytes is not None:
                kw.update(kv_cache_bytes=kv_cache_bytes, max_tokens=max_requests * per_request)
            elif torch.device(device).type == "cuda":
                spec_hidden = getattr(cfg, "hidden_size", 4096)
                spec_vocab = getattr(cfg, "vocab_size", 1 << 17)
                workspace = max_batched_tokens * spec_hidden * 64 + 8 * max_requests * spec_vocab * 4 + (1 << 30)
                kw.update(gpu_memory_fraction=gpu_memory_fraction, workspace_bytes=workspace,
                          max_tokens=max_requests * per_request)
            else:
                kw["max_tokens"] = max_requests * min(per_request, 8192)
        if model_dir is not None:
            self.runner = ModelRunner.from_model_dir(model_dir, **kw)
        else:
            self.runner = ModelRunner.from_config(config, 0 if random_weights_seed is None else random_weights_seed, **kw)
        model = self.runner.model
        self.scheduler = Scheduler(self.runner.manager, max_batched_tokens=max_batched_tokens,
                                   max_running=max_requests, chunk_size=chunk_size, max_model_len=model.max_positions)
        self.sampler = Sampler(model.spec.vocab_size, max_requests, model.device)
        self._ids = itertools.count()
        self._live: dict[object, Request] = {}
        self.pipelined = pipelined
        self._inflight: Optional[_InFlight] = None
        self._finished_early: list[GenerationResult] = []
        pin = torch.cuda.is_available() and model.device.type == "cuda"
        self._token_buffers = [torch.zeros(max_requests, dtype=torch.int32, pin_memory=pin) for _ in range(3)]
        self._token_turn = 0

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
        self._live[rid] = req      # its row of token counts (penalties) is taken when it is first scheduled
        return rid

    def abort(self, request_id) -> Optional[GenerationResult]:
        """Ends a request at once: its pages, its slot and its row of token counts are free for the
        next step.  Returns its result (``finish_reason`` "abort", the tokens that have reached the
        host), or None if it is not live.  A step of it that is in flight completes unnoticed."""
        r = self.scheduler.abort(request_id)
        if r is None:
            return None
        self.sampler.end_request(request_id)
        self._live.pop(request_id, None)
        return GenerationResult(r.request_id, r.prompt, list(r.output), r.finish_reason, r.preemptions)

    # ---------------------------------------------------------------------- step
    def _launch(self, plan: StepPlan) -> Optional[_InFlight]:
        """Builds the plan's batch, runs the model and the sampler, and starts the copy of
        the sampled tokens to the host.  Does not wait for anything."""
        prev = self._inflight

        def on_device(s) -> bool:
            """The portion's one unread token can be taken from the step in flight."""
            return s.count == 1 and prev is not None and s.request.request_id in prev.row_of

        if any(Scheduler.PLACEHOLDER in s.request.token_slice(s.start, s.count) and not on_device(s)
               for s in plan.scheduled):
            # a longer portion holds a token the host has not read yet: read the step in flight first,
            # before any entry is built, and drop what that ended (its pages are already given back)
            self._finished_early += self._resolve()
            prev = None
            plan.scheduled[:] = [s for s in plan.scheduled if s.request.status != "finished"]
        entries, rows = [], []
        for s in plan.scheduled:
            r = s.request
            toks = r.token_slice(s.start, s.count)
            src = prev.row_of[r.request_id] if Scheduler.PLACEHOLDER in toks else None   # taken on the device
            if r.params.has_penalties and not self.sampler.has_request(r.request_id):
                self.sampler.begin_request(r.request_id, r.params, r.prompt)   # admitted: at most max_requests hold a row
            entries.append(StepEntry(r.request_id, toks, [s.count - 1] if s.samples else [], token_src=src))
            if s.samples:
                rows.append(r)
        if not entries:
            return _InFlight(plan, None, None, None, {})
        prev_tokens = prev.tokens_dev if prev is not None else None
        if rows and self.sampler.all_greedy([r.params for r in rows]):
            logits, greedy_ids = self.runner.step_argmax(entries, prev_tokens=prev_tokens)
        else:
            logits, greedy_ids = self.runner.step(entries, prev_tokens=prev_tokens), None
        if not rows:
            return _InFlight(plan, None, None, None, {})
        tokens = self.sampler.sample(logits, [r.request_id for r in rows], [r.params for r in rows],
                                     [len(r.output) for r in rows], greedy_ids=greedy_ids)
        host = self._token_buffers[self._token_turn % len(self._token_buffers)]
        self._token_turn += 1
        host[:len(rows)].copy_(tokens, non_blocking=True)     # the step's one read back to the host
        done = torch.cuda.Event() if tokens.is_cuda else None
        if done is not None:
            done.record()
        return _InFlight(plan, tokens, host[:len(rows)], done, {r.request_id: i for i, r in enumerate(rows)})

    def _resolve(self) -> list[GenerationResult]:
        """Waits for the tokens of the step in flight and hands them to the scheduler."""
        fl, self._inflight = self._inflight, None
        if fl is None:
            return []
        sampled: list[int] = []
        if fl.tokens_host is not None:
            if fl.done is not None:
                fl.done.synchronize()
            sampled = fl.tokens_host.tolist()
        # a kernel whose bounded wait ran out must not pass unnoticed: checked when a request ends
        # and every 256 steps (the read of the status word waits for the device)
        self._resolved_steps = getattr(self, "_resolved_steps", 0) + 1
        finished = self.scheduler.resolve(fl.plan, sampled)
        if (finished or self._resolved_steps % 256 == 0) and self.runner.device.type == "cuda":
            ops.require_kernel_status_ok("Engine.step")
        out = []
        for r in finished:
            self.sampler.end_request(r.request_id)
            self._live.pop(r.request_id, None)
            out.append(GenerationResult(r.request_id, r.prompt, list(r.output), r.finish_reason, r.preemptions))
        return out

    def step(self) -> list[GenerationResult]:
        """One scheduler decision and one step of the model.  With ``pipelined`` (the
        default) the step is launched before the tokens of the step before it have been
        read: decoded tokens are fed on the device, the host prepares the next batch while
        the GPU works, and requests are reported finished one call later.  Returns the
        requests that finished."""
        plan: StepPlan = self.scheduler.schedule()
        self._finished_early = []
        launched = self._launch(plan) if plan.scheduled else _InFlight(plan, None, None, None, {})
        self.scheduler.advance(plan)
        finished = self._finished_early + self._resolve()       # the step before this one
        self._inflight = launched
        if not self.pipelined or not plan.scheduled:
            finished += self._resolve()
        return finished

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    def profile(self, hbm_gbs: Optional[float] = None, bf16_tflops: Optional[float] = None):
        """``with engine.profile(...) as prof:`` times every kernel launched by the steps inside the
        block per kernel class (see :mod:`zinfer_b200.profiling`); ``prof.summary()`` or
        ``prof.dump(path)`` afterwards.  The peaks, when given, turn times into fractions of the roofline."""
        return profiling.profile(hbm_gbs, bf16_tflops)

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


    def generate_stream(self, prompt_ids: Sequence[Sequence[int]], params=None, **options):
        """As :meth:`generate`, but yields ``(index of the prompt, new token ids, result or None)``
        as tokens reach the host: ``new token ids`` continue what was yielded for that prompt
        before, and ``result`` is its :class:`GenerationResult` in the event that ends it.  A tail
        that may still grow into one of the request's stop sequences is held back until it has
        not (src/app/cli/runtime/streaming.zig:42-66 on ids)."""
        if prompt_ids and isinstance(prompt_ids[0], int):
            prompt_ids = [prompt_ids]
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompt_ids)
        if len(params) != len(prompt_ids):
            raise ValueError("one SamplingParams per prompt, or one for all")
        if options:
            params = [replace(p, **options) for p in params]
        ids = [self.add_request(p, sp) for p, sp in zip(prompt_ids, params)]
        index = {rid: i for i, rid in enumerate(ids)}
        live = {rid: self._live[rid] for rid in ids}
        shown = {rid: 0 for rid in ids}
        while self.has_unfinished():
            finished = {res.request_id: res for res in self.step()}
            for rid in list(live):
                res = finished.get(rid)
                if res is not None:
                    del live[rid]
                    yield index[rid], res.token_ids[shown[rid]:], res
                    continue
                out = live[rid].output
                known = next((i for i, t in enumerate(out) if t == Scheduler.PLACEHOLDER), len(out))
                upto = analyze_generated(out[:known], live[rid].params.stop_sequences or ()).printable_len
                if upto > shown[rid]:
                    yield index[rid], list(out[shown[rid]:upto]), None
                    shown[rid] = upto


def generate(model_dir: str, prompt_ids, params: Optional[SamplingParams] = None, *, dtype="bfloat16",
             engine_options: Optional[dict] = None, **options) -> list[GenerationResult]:
    """One-call form: build an :class:`Engine` for ``model_dir`` and generate."""
    return Engine(model_dir, dtype=dtype, **(engine_options or {})).generate(prompt_ids, params, **options)
