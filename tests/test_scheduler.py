"""The scheduler's decisions (no GPU): admission, portions under a token budget,
decoding, finishing and freeing, and what happens when pages run out.  A fake step
function stands for the model: it commits the fed tokens and 'samples' a token that
is a pure function of the request and its length, as the real sampler's draws are."""
import pytest

from zinfer_b200.cache import CacheManager
from zinfer_b200.engine.scheduler import Request, Scheduler
from zinfer_b200.parts import KVCacheNeed
from zinfer_b200.sampling import SamplingParams


def make(num_pages, page=4, budget=16, chunk=None, max_running=4):
    cache = CacheManager({"l0": KVCacheNeed(1, 16, None)}, [], page, num_pages, max_running)
    return cache, Scheduler(cache, max_batched_tokens=budget, max_running=max_running, chunk_size=chunk)


def fake_token(r: Request) -> int:
    import zlib
    return (zlib.crc32(repr(r.request_id).encode()) + 7 * r.num_tokens) % 97 + 3


def run_step(cache, sched, log=None):
    plan = sched.schedule()
    sampled = []
    for s in plan.scheduled:
        assert cache.length(s.request.request_id) == s.start, "the fed portion does not continue the cache"
        cache.commit(s.request.request_id, s.count)
        if s.samples:
            sampled.append(fake_token(s.request))
    if log is not None:
        log.append([(s.request.request_id, s.start, s.count, s.samples) for s in plan.scheduled])
    done = sched.update(plan, sampled)
    cache.check()
    return plan, done


def drain(cache, sched, limit=2000):
    done, log = [], []
    while sched.has_unfinished():
        limit -= 1
        assert limit > 0, "the scheduler does not terminate"
        done += run_step(cache, sched, log)[1]
    return done, log


def req(rid, n_prompt, max_new, **kw):
    return Request(rid, list(range(1, n_prompt + 1)), SamplingParams(temperature=0.0, max_new_tokens=max_new, **kw))


def test_prompts_are_cut_under_the_budget_and_decodes_go_first():
    cache, sched = make(num_pages=64, budget=16, chunk=10)
    sched.add(req("a", 23, 3))
    sched.add(req("b", 5, 2))
    log = []
    run_step(cache, sched, log)
    assert log[-1] == [("a", 0, 10, False), ("b", 0, 5, True)]        # chunk 10, then b whole within the budget of 16
    run_step(cache, sched, log)
    assert log[-1] == [("b", 5, 1, True), ("a", 10, 10, False)]       # b decodes first, a's next portion after
    run_step(cache, sched, log)
    assert log[-1][0] == ("a", 20, 3, True)                           # the last portion samples; b ended after 2 tokens
    done, _ = drain(cache, sched)
    assert not sched.has_unfinished() and cache.free_pages() == [64] and not cache.requests


def test_budget_is_never_exceeded_and_portions_can_be_tiny():
    cache, sched = make(num_pages=200, budget=7, max_running=4)
    for i in range(6):
        sched.add(req(i, 9 + i, 4))
    done, log = drain(cache, sched)
    assert len(done) == 6 and all(r.finish_reason == "length" and len(r.output) == 4 for r in done)
    assert all(sum(c for _, _, c, _ in step) <= 7 for step in log)
    assert any(c <= 2 and not s for step in log for _, _, c, s in step), "no small portion was ever cut"
    assert max(len(step) for step in log) <= 4


def test_finishing_frees_pages_and_admits_the_next():
    cache, sched = make(num_pages=4, page=4, budget=64, max_running=4)   # 16 tokens of cache in all
    sched.add(req("a", 10, 2))
    sched.add(req("b", 10, 2))
    plan, _ = run_step(cache, sched)
    assert [s.request.request_id for s in plan.scheduled] == ["a", "b"]
    assert plan.scheduled[1].count == 4 and not plan.scheduled[1].samples   # b's portion is cut to the free page
    done, log = drain(cache, sched)
    assert {r.request_id for r in done} == {"a", "b"} and all(len(r.output) == 2 for r in done)
    assert cache.free_pages() == [4]


def test_eos_ends_a_request_and_is_not_emitted():
    cache, sched = make(num_pages=16)
    r = req("a", 3, 50)
    plan = None
    sched.add(r)
    r.eos_token_ids = (fake_token(Request("a", [0] * 5, r.params)),)     # the token 'sampled' at length 5
    done, _ = drain(cache, sched)
    assert done[0].finish_reason == "stop" and len(done[0].output) == 2
    cache2, sched2 = make(num_pages=16)
    r2 = req("a", 3, 4, ignore_eos=True)
    r2.eos_token_ids = r.eos_token_ids
    sched2.add(r2)
    done2, _ = drain(cache2, sched2)
    assert done2[0].finish_reason == "length" and len(done2[0].output) == 4


def test_out_of_pages_preempts_the_latest_admitted_and_output_is_unchanged():
    def outputs(num_pages):
        cache, sched = make(num_pages=num_pages, page=4, budget=64, max_running=3)
        for i, n in enumerate((6, 7, 5)):
            sched.add(req(i, n, 12))
        done, log = drain(cache, sched)
        return {r.request_id: (r.output, r.finish_reason, r.preemptions) for r in done}, sched.stats, log

    roomy, st_roomy, _ = outputs(64)
    tight, st_tight, log = outputs(9)       # 36 tokens of cache for 3 requests growing to 18, 19 and 17
    assert st_roomy.preemptions == 0 and st_tight.preemptions > 0
    assert {k: v[:2] for k, v in tight.items()} == {k: v[:2] for k, v in roomy.items()}, \
        "preemption and recomputation changed a request's tokens"
    assert tight[0][2] == 0, "the oldest request must never be preempted"
    assert any(v[2] > 0 for v in tight.values())
    # a preempted request starts again from position 0 with its generated tokens as part of the prompt
    restarts = [e for step in log for e in step if e[1] == 0]
    assert len(restarts) > 3


def test_request_larger_than_the_pool_ends_with_capacity():
    cache, sched = make(num_pages=2, page=4, budget=64)
    sched.add(req("big", 5, 10))           # 8 tokens of cache: the prompt fits, decoding outgrows the pool
    sched.add(req("huge", 20, 2))          # its prompt alone is larger than the pool
    done, _ = drain(cache, sched)
    by = {r.request_id: r for r in done}
    assert by["big"].finish_reason == "capacity" and len(by["big"].output) == 4   # 5 + 3 fed tokens fill the 8 slots
    assert by["huge"].finish_reason == "capacity" and by["huge"].output == []
    assert cache.free_pages() == [2] and not cache.requests


def test_waiting_requests_keep_their_order():
    cache, sched = make(num_pages=64, budget=8, max_running=2)
    for i in range(5):
        sched.add(req(i, 4, 3))
    _, log = drain(cache, sched)
    first_seen = []
    for step in log:
        for rid, start, _, _ in step:
            if start == 0 and rid not in first_seen:
                first_seen.append(rid)
    assert first_seen == [0, 1, 2, 3, 4]
    assert max(len(step) for step in log) <= 2


def drain_pipelined(cache, sched, limit=2000, plans=None):
    """The engine's pipelined order: a step is launched (advance) before the tokens of the
    step before it are read (resolve), so end-of-sequence is noticed one step late."""
    done, pending = [], None
    while sched.has_unfinished() or pending is not None:
        limit -= 1
        assert limit > 0
        plan = sched.schedule()
        if plans is not None:
            plans.append(plan)
        sampled = []
        for s in plan.scheduled:
            assert cache.length(s.request.request_id) == s.start
            cache.commit(s.request.request_id, s.count)
            if s.samples:
                # the fake token depends on the request and its length only, like a seeded draw
                r = s.request
                sampled.append(fake_token(Request(r.request_id, [0] * (s.start + s.count), r.params)))
        sched.advance(plan)
        if pending is not None:
            done += sched.resolve(*pending)
        pending = (plan, sampled) if plan.scheduled else None
        if not plan.scheduled:
            done += sched.resolve(plan, [])
        cache.check()
    return done


def test_pipelined_resolution_gives_the_same_tokens_and_reasons():
    def build(num_pages):
        cache, sched = make(num_pages=num_pages, page=4, budget=32, max_running=3)
        reqs = [req(i, n, 10) for i, n in enumerate((6, 7, 5, 9))]
        # request 1 stops at its 4th token, request 3 at its 1st
        reqs[1].eos_token_ids = (fake_token(Request(1, [0] * (7 + 3), reqs[1].params)),)
        reqs[3].eos_token_ids = (fake_token(Request(3, [0] * 9, reqs[3].params)),)
        for r in reqs:
            sched.add(r)
        return cache, sched

    for pages in (64, 9):
        cache, sched = build(pages)
        sync, _ = drain(cache, sched)
        cache2, sched2 = build(pages)
        piped = drain_pipelined(cache2, sched2)
        key = lambda rs: sorted((r.request_id, tuple(r.output), r.finish_reason) for r in rs)
        assert key(piped) == key(sync)
        assert all(-1 not in r.output for r in piped), "a placeholder was left in an output"
        by = {r.request_id: r for r in piped}
        assert by[1].finish_reason == "stop" and len(by[1].output) == 3
        assert by[3].finish_reason == "stop" and by[3].output == []
        assert by[0].finish_reason == "length" and len(by[0].output) == 10
        assert not cache2.requests and cache2.free_pages() == [pages]


def test_end_of_sequence_in_flight_when_the_request_is_preempted():
    """A request draws its end-of-sequence token in step k; before the host has read that token,
    step k+1's schedule preempts the request (an older one needs its page).  It must be reported
    once, with reason stop, hold no placeholder, and never be admitted again."""
    def build(eos_for_b=()):
        cache, sched = make(num_pages=6, page=4, budget=32, max_running=2)
        a, b = req("a", 7, 12, ignore_eos=True), req("b", 6, 12)
        b.eos_token_ids = tuple(eos_for_b)
        sched.add(a)
        sched.add(b)
        return cache, sched, b

    # first without an end token: find the step whose schedule preempts b, and the token b drew
    # in the step before it (a function of its length, like a seeded draw)
    cache, sched, b = build()
    plans = []
    drain_pipelined(cache, sched, plans=plans)
    k1 = next(i for i, p in enumerate(plans) if any(r is b for r in p.preempted))
    before = next(s for s in plans[k1 - 1].scheduled if s.request is b)
    assert before.samples, "the case is meant to have b's token in flight when it is preempted"
    eos = fake_token(Request("b", [0] * (before.start + before.count), b.params))
    n_out = before.start + before.count - 6      # tokens b had emitted before that one

    cache, sched, b = build([eos])
    plans = []
    done = drain_pipelined(cache, sched, plans=plans)
    assert any(r is b for r in plans[k1].preempted), "the end token did not change the schedule before it was read"
    reports = [r for r in done if r is b]
    assert len(reports) == 1, f"b was reported {len(reports)} times"
    assert b.finish_reason == "stop" and len(b.output) <= n_out and -1 not in b.output
    assert not sched.waiting and not sched.running and not cache.requests and cache.free_pages() == [6]
    assert all(all(s.request is not b for s in p.scheduled) for p in plans[k1 + 1:]), "b ran again after it had ended"
    # the same tokens as a host that waits for every step
    cache2, sched2, b2 = build([eos])
    sync, _ = drain(cache2, sched2)
    key = lambda rs: sorted((r.request_id, tuple(r.output), r.finish_reason) for r in rs)
    assert key(done) == key(sync)


def test_decode_attention_split_choice():
    """The split count of the decode attention (a host decision): one wave of blocks when the
    requests are few, whole waves when they are many, never more splits than tiles of 64 keys."""
    from zinfer_b200.ops import decode_splits

    sms = 148
    assert 12 <= decode_splits(1, 8, sms, 2048) <= 20      # one request: many splits fill the GPU, but each costs its merge
    assert decode_splits(8, 8, sms, 2048) == 4             # 64 (request, head) pairs x 4 = 256 blocks on 296 slots
    assert decode_splits(32, 8, sms, 2048) == 1            # 256 pairs already fill a wave
    assert decode_splits(48, 8, sms, 2048) == 1            # 384 pairs: more than half a wave of few keys is never split
    assert decode_splits(64, 8, sms, 16384) > 1            # long walks: whole waves matter more than the merge
    assert decode_splits(8, 8, sms, 100) <= 2              # 100 keys are two tiles of 64
    assert decode_splits(8, 8, sms, 0) >= 1 and decode_splits(8, 8, sms, None) >= 1
    for n in range(1, 130):
        for keys in (1, 63, 64, 65, 1000, 8192):
            s = decode_splits(n, 8, sms, keys)
            assert 1 <= s <= 32 and s <= max(1, -(-keys // 64))
