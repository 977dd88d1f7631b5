"""The scheduler above the step function: continuous batching with prompts cut
into portions under a token budget.

Every step it decides, in this order:

1. each running request whose prompt is in the cache gets its one next token;
2. running requests still in their prompt get the next portion;
3. waiting requests are admitted, oldest first, while a request slot, pages for a
   first portion and budget remain.

A portion is ``min(tokens left, chunk_size, budget left)`` and may be as small as
one token.  A request's tokens are its prompt followed by what it has generated;
``num_computed`` of them are in the cache, so prompt portions, decoding and
recomputation after preemption are one case.

When pages run out:

* a request that needs a page for its next decoded token takes it from the running
  request admitted last (never from an older one): that request is *preempted*, all
  its pages are given back and it returns to the front of the waiting queue; when it
  is admitted again its prompt and the tokens it had generated are recomputed, and
  because the i-th draw depends only on (seed, i) its output is unchanged;
* a prompt portion that does not fit is shortened to the pages that are free, or
  waits for a later step; it never preempts;
* a request that is alone and still cannot get a page is finished with the reason
  ``capacity``: the pool is too small for it.

The reference has fixed slots, whole blocking prefills and no page allocator
(src/model/runtime/optimized_decoder/batch.zig:92-209); finishing follows it: an
end-of-sequence token is neither emitted nor fed (src/app/cli/runtime/generator.zig:103-105),
and a request ends after ``max_new_tokens`` (batch.zig:131-135).

Host code only: it imports no device code and is tested without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams
from ..sampling.stop import stop_hit_at


@dataclass(eq=False)      # a request is itself, never "equal" to another: queues compare by identity
class Request:
    request_id: Hashable
    prompt: list[int]
    params: SamplingParams
    eos_token_ids: tuple[int, ...] = ()
    output: list[int] = field(default_factory=list)
    num_computed: int = 0            # tokens of prompt + output that are in the cache
    status: str = "waiting"          # waiting | running | finished
    finish_reason: Optional[str] = None   # stop (end-of-sequence) | length | capacity
    admitted_at: int = -1            # admission counter; larger = admitted later
    preemptions: int = 0

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_slice(self, start: int, count: int) -> list[int]:
        """``tokens[start:start + count]`` without joining prompt and output first."""
        n = len(self.prompt)
        end = start + count
        if end <= n:
            return self.prompt[start:end]
        if start >= n:
            return self.output[start - n:end - n]
        return self.prompt[start:] + self.output[:end - n]


@dataclass
class Scheduled:
    request: Request
    start: int                       # index of the first token fed, into request.tokens
    count: int
    samples: bool                    # the last fed token is the request's last: its logits are sampled


@dataclass
class StepPlan:
    scheduled: list[Scheduled] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)
    finished: list[Request] = field(default_factory=list)   # ended by the scheduler itself (capacity, length)

    @property
    def num_tokens(self) -> int:
        return sum(s.count for s in self.scheduled)


@dataclass
class SchedulerStats:
    """Totals since the scheduler was made, and the state after the last ``schedule()``."""

    steps: int = 0
    prompt_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    # the last step
    step_tokens: int = 0          # tokens scheduled in it
    running: int = 0
    waiting: int = 0
    pages_used: int = 0           # in the fullest cache group
    pages_total: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, max_batched_tokens: int = 2048, max_running: int = 64,
                 chunk_size: Optional[int] = None, max_model_len: int = 1 << 30):
        if max_batched_tokens <= 0:
            raise ValueError("max_batched_tokens must be positive")
        self.cache = cache
        self.max_batched_tokens = max_batched_tokens
        self.max_running = min(max_running, cache.max_requests)
        self.chunk_size = chunk_size or max_batched_tokens
        self.max_model_len = max_model_len
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []          # in admission order
        self.stats = SchedulerStats()
        self._admissions = 0

    # ------------------------------------------------------------------ requests
    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise ValueError(f"request {request.request_id!r} has an empty prompt")
        request.status = "waiting"
        self.waiting.append(request)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, request_id: Hashable) -> Optional[Request]:
        """Ends a waiting or running request now (``finish_reason`` "abort") and gives back what it
        holds; the request is returned with the tokens that have reached the host.  A token of it
        that is still in flight is dropped when its step is resolved.  None if no such request lives."""
        r = next((x for x in list(self.running) + list(self.waiting) if x.request_id == request_id), None)
        if r is None:
            return None
        known = next((i for i, t in enumerate(r.output) if t == self.PLACEHOLDER), len(r.output))
        del r.output[known:]
        self._finish(r, "abort")
        return r

    # -------------------------------------------------------------------- helpers
    def _release(self, r: Request) -> None:
        if self.cache.has_request(r.request_id):
            self.cache.free_request(r.request_id)

    def _finish(self, r: Request, reason: str, plan: Optional[StepPlan] = None) -> None:
        r.status, r.finish_reason = "finished", reason
        self._release(r)
        if r in self.running:
            self.running.remove(r)
        if r in self.waiting:
            # preempted while the token that ends it was still in flight: it must not be admitted again
            self.waiting.remove(r)
        self.stats.finished += 1
        if plan is not None:
            plan.finished.append(r)

    def _preempt(self, r: Request, plan: StepPlan) -> None:
        self._release(r)
        self.running.remove(r)
        r.status, r.num_computed = "waiting", 0
        r.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(r)
        plan.preempted.append(r)

    def _fit(self, r: Request, want: int) -> int:
        """The most tokens <= want whose pages are free right now."""
        if self.cache.can_reserve(r.request_id, want):
            return want
        ps = self.cache.page_size
        have = self.cache.blocks_held(r.request_id) * ps if self.cache.groups else 1 << 30
        room = have + self.cache.min_free_pages() * ps - self.cache.length(r.request_id)
        return max(0, min(want, room))

    # ------------------------------------------------------------------- schedule
    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_batched_tokens
        taken: set = set()

        # 1. one token for every running request that is decoding
        for r in list(self.running):
            if r.status != "running" or r.num_tokens - r.num_computed != 1 or not r.output:
                continue
            if budget <= 0:
                break
            while not self.cache.can_reserve(r.request_id, 1):
                victim = next((v for v in reversed(self.running) if v is not r and id(v) not in taken), None)
                if victim is None or victim.admitted_at < r.admitted_at:
                    break
                self._preempt(victim, plan)
            if r.status != "running":
                continue
            if not self.cache.can_reserve(r.request_id, 1):
                others = [v for v in self.running if v is not r]
                if not others:
                    self._finish(r, "capacity", plan)   # alone, and the pool is too small for it
                continue                                 # else: an older request holds the pages; wait
            self.cache.reserve(r.request_id, 1)
            plan.scheduled.append(Scheduled(r, r.num_computed, 1, samples=True))
            taken.add(id(r))
            budget -= 1

        # 2. the next portion of running requests still in their prompt (or recomputing)
        for r in list(self.running):
            if id(r) in taken or r.status != "running" or budget <= 0:
                continue
            left = r.num_tokens - r.num_computed
            n = self._fit(r, min(left, self.chunk_size, budget))
            if n <= 0:
                continue
            self.cache.reserve(r.request_id, n)
            plan.scheduled.append(Scheduled(r, r.num_computed, n, samples=(n == left)))
            taken.add(id(r))
            budget -= n

        # 3. admissions, oldest first; none may overtake a request that does not fit
        while self.waiting and budget > 0 and len(self.running) < self.max_running and not plan.preempted:
            r = self.waiting[0]
            assert r.status == "waiting", f"request {r.request_id!r} is {r.status} but still queued"
            if r.num_tokens >= self.max_model_len or r.params.max_new_tokens <= len(r.output):
                self.waiting.popleft()
                self._finish(r, "length", plan)
                continue
            self.cache.add_request(r.request_id)
            n = self._fit(r, min(r.num_tokens, self.chunk_size, budget))
            if n <= 0:
                self.cache.free_request(r.request_id)
                if not self.running:
                    self.waiting.popleft()
                    self._finish(r, "capacity", plan)   # nothing else holds pages: it can never start
                    continue
                break
            self.waiting.popleft()
            self.cache.reserve(r.request_id, n)
            r.status = "running"
            r.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(r)
            plan.scheduled.append(Scheduled(r, 0, n, samples=(n == r.num_tokens)))
            budget -= n

        # a running prompt that cannot advance while nobody else runs would wait for ever
        if not plan.scheduled and not plan.finished and self.running:
            stuck = self.running[-1]
            if len(self.running) == 1:
                self._finish(stuck, "capacity", plan)
            else:
                self._preempt(stuck, plan)
        st = self.stats
        st.steps += 1
        st.step_tokens, st.running, st.waiting = plan.num_tokens, len(self.running), len(self.waiting)
        if self.cache.groups:
            st.pages_total = self.cache.groups[0].pool.num_pages
            st.pages_used = st.pages_total - self.cache.min_free_pages()
        return plan

    # --------------------------------------------------------------------- update
    PLACEHOLDER = -1   # a token that has been sampled on the device but not yet read by the host

    def advance(self, plan: StepPlan) -> None:
        """Call when the plan's step has been launched: the fed tokens count as computed,
        every sampling request gets a placeholder for the token being sampled, and requests
        that thereby reach their length limit leave the running set (their pages are given
        back; later work on the same stream cannot overtake the step that still reads them)."""
        for s in plan.scheduled:
            r = s.request
            was_decode = s.count == 1 and s.start >= len(r.prompt)
            r.num_computed = s.start + s.count
            if was_decode:
                self.stats.decode_tokens += 1
            else:
                self.stats.prompt_tokens += s.count
            if not s.samples:
                continue
            r.output.append(self.PLACEHOLDER)
            if len(r.output) >= r.params.max_new_tokens or r.num_tokens >= self.max_model_len:
                self._finish(r, "length")

    def resolve(self, plan: StepPlan, sampled: Sequence[int]) -> list[Request]:
        """Call when the plan's sampled tokens (in plan order) have reached the host: fills
        the placeholders in, ends requests that drew an end-of-sequence token (which is
        neither emitted nor fed), and returns all requests that this plan finished."""
        finished = list(plan.finished)
        it = iter(sampled)
        for s in plan.scheduled:
            if not s.samples:
                continue
            r = s.request
            tok = int(next(it))
            if r.finish_reason in ("stop", "abort"):
                continue                                 # ended by an earlier token, or aborted; this one is dropped
            idx = s.start + s.count - len(r.prompt)      # which output this step sampled
            if not r.params.ignore_eos and tok in r.eos_token_ids:
                del r.output[idx:]                       # the end token and anything in flight after it
                if r.status != "finished":
                    self._finish(r, "stop")
                else:                                    # had also reached its length limit with this token
                    r.finish_reason = "stop"
                finished.append(r)
                continue
            if idx < len(r.output):
                r.output[idx] = tok
                hit = stop_hit_at(r.output, idx + 1, r.params.stop_sequences) if r.params.stop_sequences else 0
                if hit:
                    del r.output[idx + 1 - hit:]         # the stop sequence and anything in flight after it
                    if r.status != "finished":
                        self._finish(r, "stop")
                    else:
                        r.finish_reason = "stop"
                    finished.append(r)
                    continue
            if r.status == "finished" and r.finish_reason == "length" and idx == len(r.output) - 1:
                finished.append(r)
        return finished

    def update(self, plan: StepPlan, sampled: Sequence[int]) -> list[Request]:
        """The two phases back to back, for a host that waits for each step's tokens."""
        self.advance(plan)
        return self.resolve(plan, sampled)
