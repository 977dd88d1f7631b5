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
