"""The entry point's host logic without a GPU (the kernels replaced by their plain
references): end-of-sequence noticed one step late, token-count rows for penalties,
and pipelined against unpipelined operation."""
import pytest

import plain_qwen3 as P
from conftest import PAGE_SIZE


def _engine(model_dirs, name, **kw):
    from zinfer_b200.engine.api import Engine

    opts = dict(dtype="float32", device="cpu", page_size=PAGE_SIZE[name], kv_cache_tokens=512, max_batched_tokens=16,
                max_requests=4)
    opts.update(kw)
    return Engine(model_dirs[(name, "float32")], **opts)


def _prompts(V, lengths=(5, 17, 33, 1, 9)):
    return [[(5 * i + 3 * j) % V for j in range(n)] for i, n in enumerate(lengths)]


@pytest.mark.parametrize("pipelined", [True, False])
def test_end_of_sequence_through_the_engine(cpu_kernels, model_dirs, pipelined):
    """Every request gets its own end token, taken from the plain model's greedy continuation, so
    that requests stop at different steps; the pool is so small that freed pages are taken at once."""
    from zinfer_b200.sampling import SamplingParams

    cfg, w = P.load_model(model_dirs[("A", "float32")])
    prompts = _prompts(cfg["vocab_size"])
    full = [P.greedy(cfg, w, p, 10) for p in prompts]
    stops = [2, 5, 0, 9, 3]          # the index of the token that ends each request
    params = [SamplingParams(temperature=0.0, max_new_tokens=10, eos_token_ids=(f[s],)) for f, s in zip(full, stops)]
    want = [f[:f.index(f[s])] for f, s in zip(full, stops)]       # cut at the first occurrence of the end token
    eng = _engine(model_dirs, "A", kv_cache_tokens=96, pipelined=pipelined)
    got = eng.generate(prompts, params)
    assert [r.token_ids for r in got] == want
    assert all(r.finish_reason == "stop" for r in got)
    eng.runner.manager.check()
    assert not eng.runner.manager.requests and not eng.scheduler.waiting and not eng.scheduler.running


def test_more_penalised_prompts_than_count_rows(cpu_kernels, model_dirs):
    """A row of token counts is taken when a request is admitted, not when it is queued: more
    queued prompts with penalties than rows must not fail, and every row is given back."""
    from zinfer_b200.sampling import SamplingParams

    eng = _engine(model_dirs, "A", max_requests=2)
    sp = SamplingParams(temperature=0.7, top_k=8, repetition_penalty=1.3, presence_penalty=0.1, seed=3, max_new_tokens=4,
                        ignore_eos=True)
    prompts = _prompts(256, (4, 9, 3, 7, 5))
    got = eng.generate(prompts, sp)
    assert all(len(r.token_ids) == 4 for r in got)
    assert eng.sampler._rows.num_used == 0 and not eng.sampler._row_of
    alone = [_engine(model_dirs, "A", max_requests=2).generate([p], sp)[0].token_ids for p in prompts]
    assert [r.token_ids for r in got] == alone, "a request's tokens depend on what ran beside it"


def test_stop_analysis_on_ids():
    """The reference's two cases (src/app/cli/runtime/streaming.zig:68-87) with ids for bytes, and
    the order of several stop sequences."""
    from zinfer_b200.sampling import analyze_generated

    hello_today = [7, 4, 11, 11, 14, 99, 19, 14, 3, 0, 24, 50]      # "Hello today?"
    today = hello_today[6:]
    a = analyze_generated(hello_today, [today])
    assert (a.stop_hit, a.printable_len, a.response_len) == (True, 6, 6)
    a = analyze_generated(hello_today[:8], [today])                 # "Hello to": a prefix of the stop is held back
    assert (a.stop_hit, a.printable_len, a.response_len) == (False, 6, 8)
    a = analyze_generated([1, 2, 3], [[], [9], [2, 3, 4], [3, 5, 5]])
    assert (a.stop_hit, a.printable_len, a.response_len) == (False, 1, 3)   # the longest tail that may still grow
    a = analyze_generated([1, 2, 3], [[3], [2, 3]])
    assert (a.stop_hit, a.response_len) == (True, 2)                # the first sequence that matches, in the order given
    assert analyze_generated([], [[1]]) == analyze_generated([], [])


@pytest.mark.parametrize("pipelined", [True, False])
def test_stop_sequences_and_streaming_through_the_engine(cpu_kernels, model_dirs, pipelined):
    """Stop sequences cut from the plain greedy continuation: the response ends before the
    sequence, whatever was in flight is dropped, and the streamed pieces add up to the response
    without ever showing a tail that became a stop sequence."""
    from zinfer_b200.sampling import SamplingParams

    cfg, w = P.load_model(model_dirs[("A", "float32")])
    prompts = _prompts(cfg["vocab_size"])
    full = [P.greedy(cfg, w, p, 12) for p in prompts]
    # request i stops on the two ids at positions cut[i], cut[i]+1 of its continuation; the last has a
    # stop sequence that never occurs, and one whose first id alone occurs (held back, then shown)
    cut = [3, 0, 7, 10]
    params = [SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True, stop_sequences=[[4242, 1], f[c:c + 2]])
              for f, c in zip(full, cut)]
    params.append(SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True,
                                 stop_sequences=[[full[4][5], cfg["vocab_size"] + 5]]))
    def first_hit(f, stop):
        return next((i for i in range(len(f) - 1) if f[i:i + 2] == stop), None)
    want = [f[:first_hit(f, f[c:c + 2])] for f, c in zip(full, cut)] + [full[4]]
    eng = _engine(model_dirs, "A", kv_cache_tokens=96, pipelined=pipelined)
    got = eng.generate(prompts, params)
    assert [r.token_ids for r in got] == want
    assert [r.finish_reason for r in got] == ["stop"] * 4 + ["length"]
    eng.runner.manager.check()
    assert not eng.runner.manager.requests and not eng.scheduler.waiting and not eng.scheduler.running
    pieces = {i: [] for i in range(5)}
    ended = {}
    for i, new_ids, res in eng.generate_stream(prompts, params):
        assert i not in ended, "nothing comes after the event that ends a request"
        pieces[i] += new_ids
        assert pieces[i] == want[i][:len(pieces[i])], "a token was shown that is not part of the response"
        if res is not None:
            ended[i] = res
    assert [pieces[i] for i in range(5)] == want and [ended[i].token_ids for i in range(5)] == want


@pytest.mark.parametrize("pipelined", [True, False])
def test_abort_gives_everything_back_and_disturbs_nobody(cpu_kernels, model_dirs, pipelined):
    """A running request (with a token in flight when the engine is pipelined) and a waiting one are
    aborted between steps: their pages, slots and count rows are free at once, they are reported once,
    with the tokens that had reached the host, and the other requests' tokens are the plain model's."""
    from zinfer_b200.sampling import SamplingParams

    cfg, w = P.load_model(model_dirs[("A", "float32")])
    prompts = _prompts(cfg["vocab_size"], lengths=(5, 17, 9, 12))
    want = [P.greedy(cfg, w, p, 8) for p in prompts]
    eng = _engine(model_dirs, "A", kv_cache_tokens=96, max_requests=2, pipelined=pipelined)
    sp = SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True, repetition_penalty=1.0)
    pen = SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True, presence_penalty=1e-9)   # takes a count row
    ids = [eng.add_request(p, pen if i == 1 else sp) for i, p in enumerate(prompts)]
    done = {}
    for _ in range(4):                                   # requests 0 and 1 run, 2 and 3 wait
        for res in eng.step():
            done[res.request_id] = res
    assert [r.request_id for r in eng.scheduler.running] == ids[:2] and len(eng.scheduler.waiting) == 2
    a = eng.abort(ids[1])
    b = eng.abort(ids[3])
    assert eng.abort(ids[1]) is None and eng.abort("nobody") is None
    assert a.finish_reason == b.finish_reason == "abort" and b.token_ids == []
    assert -1 not in a.token_ids and a.token_ids == want[1][:len(a.token_ids)] and 0 < len(a.token_ids) < 8
    assert not eng.runner.manager.has_request(ids[1]) and not eng.sampler.has_request(ids[1])
    while eng.has_unfinished():
        for res in eng.step():
            assert res.request_id not in (ids[1], ids[3]), "an aborted request was reported again"
            done[res.request_id] = res
    assert done[ids[0]].token_ids == want[0] and done[ids[2]].token_ids == want[2]
    eng.runner.manager.check()
    assert not eng.runner.manager.requests and not eng.scheduler.waiting and not eng.scheduler.running
