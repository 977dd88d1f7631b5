"""The whole engine on the GPU: generation through the entry point and the command
line, long decoding, the first tokens of a sequence, sampling, and each part alone."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kernel_refs as ref
import plain_qwen3 as P
import replay_util as ru
from conftest import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _engine(d, name, dtype, **kw):
    from zinfer_b200.engine.api import Engine

    opts = dict(dtype=dtype, device=DEV, page_size=PAGE_SIZE[name], kv_cache_tokens=1024, max_batched_tokens=16,
                max_requests=4)
    opts.update(kw)
    return Engine(d, **opts)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_generation_through_the_entry_point(model_dirs, name):
    from zinfer_b200.sampling import SamplingParams

    d = model_dirs[(name, "float32")]
    cfg, w = P.load_model(d)
    V = cfg["vocab_size"]
    prompts = [[(5 * i + 3 * j) % V for j in range(n)] for i, n in enumerate((5, 17, 33, 1, 9))]
    want = [P.greedy(cfg, w, p, 16) for p in prompts]
    eng = _engine(d, name, "float32")
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=16, ignore_eos=True))
    assert [r.token_ids for r in got] == want
    # bfloat16: every chosen token must be (nearly) the best one under the plain model given the same history
    d16 = model_dirs[(name, "bfloat16")]
    cfg16, w16 = P.load_model(d16)
    got16 = _engine(d16, name, "bfloat16").generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=16, ignore_eos=True))
    for p, r in zip(prompts, got16):
        assert len(r.token_ids) == 16
        logits = P.forward(cfg16, w16, p + r.token_ids).numpy()
        for i, t in enumerate(r.token_ids):
            row = logits[len(p) - 1 + i]
            assert row[t] >= row.max() - 3e-2 * np.abs(row).max(), f"bfloat16 picked token {t} far from the best"


def test_tight_pool_preempts_and_keeps_the_tokens(model_dirs):
    from zinfer_b200.sampling import SamplingParams

    d = model_dirs[("A", "float32")]
    cfg, w = P.load_model(d)
    prompts = [[(7 * i + j) % 200 + 1 for j in range(15 - i)] for i in range(3)]
    want = [P.greedy(cfg, w, p, 8) for p in prompts]
    eng = _engine(d, "A", "float32", kv_cache_tokens=None, num_pages=4)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))
    assert [r.token_ids for r in got] == want
    assert eng.scheduler.stats.preemptions > 0
    eng.runner.manager.check()


def test_command_line_generate_token_ids(model_dirs):
    d = model_dirs[("B", "float32")]
    cfg, w = P.load_model(d)
    r = subprocess.run([sys.executable, os.path.join(REPO, "bin", "zinfer"), "generate-token-ids", d, "5,17,3", "6",
                        "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    want = [5, 17, 3] + P.greedy(cfg, w, [5, 17, 3], 6)
    assert "tokens: [" + ", ".join(map(str, want)) + "]" in r.stdout
    assert "Zinfer generated token ids" in r.stdout and "steps: 6" in r.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(model_dirs, dtype):
    """A one-token prompt, then 400 tokens decoded one by one (far past several pages),
    against the plain model on the whole sequence."""
    from zinfer_b200.engine import ModelRunner

    d = model_dirs[("C", dtype)]
    cfg, w = P.load_model(d)
    reqs = ru.make_requests(cfg["vocab_size"], [401], seed=3)
    toks = reqs["r0"]
    trace = [{"step": i, "entries": [{"id": "r0", "tokens": toks[i:i + 1], "want": [0]}], "end": []} for i in range(401)]
    runner = ModelRunner.from_model_dir(d, dtype=getattr(torch, dtype), device=DEV, page_size=32, max_tokens=448)
    got = ru.run_in_process_keep(runner, trace) if hasattr(ru, "run_in_process_keep") else None
    if got is None:
        trace[-1]["end"] = ["r0"]
        got = ru.run_in_process(runner, trace)
    tol = dict(rtol=5e-5, atol=1e-6) if dtype == "float32" else dict(rtol=3e-2, atol=1e-3)
    ru.assert_close(got, ru.plain_logits(cfg, w, reqs), what=f"long decode {dtype}", argmax_frac=0.0, **tol)
    first = {k: v for k, v in got.items() if k[1] < 3}
    assert len(first) == 3


# ----------------------------------------------------------------------- sampling
def _sample_many(logits_row, n, **kw):
    from zinfer_b200 import ops

    V = logits_row.numel()
    logits = logits_row.to(DEV).float().unsqueeze(0).repeat(n, 1).contiguous()
    f = lambda v: torch.full((n,), v, dtype=torch.float32, device=DEV)
    i = lambda v: torch.full((n,), v, dtype=torch.int32, device=DEV)
    return ops.sample(logits, temperature=f(kw.get("temperature", 1.0)), seeds=torch.full((n,), kw.get("seed", 5), dtype=torch.int64, device=DEV),
                      draw_index=torch.arange(n, dtype=torch.int32, device=DEV), top_k=i(kw.get("top_k", 0)),
                      top_p=f(kw.get("top_p", 1.0)), min_p=f(kw.get("min_p", 0.0))).cpu().numpy()


@pytest.mark.parametrize("kw", [dict(temperature=0.8), dict(temperature=1.3, top_k=20), dict(temperature=0.7, top_k=20, top_p=0.8),
                                dict(temperature=1.0, min_p=0.2), dict(temperature=0.6, top_p=0.95, top_k=50, min_p=0.05)])
def test_sampling_follows_the_kept_distribution(kw):
    V, n = 1000, 20000
    g = torch.Generator().manual_seed(0)
    row = torch.randn(V, generator=g) * 2.0
    row[17] = row[400] = row.max()   # a tie at the top
    draws = _sample_many(row, n, **kw)
    p = P.kept_distribution(row.numpy(), kw["temperature"], kw.get("top_k", 0), kw.get("top_p", 1.0), kw.get("min_p", 0.0))
    freq = np.bincount(draws, minlength=V) / n
    assert set(np.nonzero(freq)[0]) <= set(np.nonzero(p)[0]), "a token outside the kept set was drawn"
    big = p > 0.01
    np.testing.assert_allclose(freq[big], p[big], atol=4 * np.sqrt(p[big].max() / n) + 2e-3)
    assert abs(freq[~big].sum() - p[~big].sum()) < 0.02
    again = _sample_many(row, n, **kw)
    assert (again == draws).all(), "the same seed and draw index gave another token"
    other = _sample_many(row, n, **{**kw, "seed": 6})
    assert (other != draws).any()


@pytest.mark.parametrize("V", [1000, 151936])
def test_a_draw_does_not_depend_on_the_rows_beside_it(V):
    """The kernel spreads a row over 8, 4, 2 or 1 CTAs by the number of rows in the launch; the
    token drawn for a row must be the same in every case, for each of the kernel's routes (few
    candidates listed and sorted, many candidates cut by thresholds, with and without penalties)."""
    from zinfer_b200 import ops

    g = torch.Generator().manual_seed(3)
    base = (torch.randn(12, V, generator=g) * 2.5).to(DEV)
    counts_base = (torch.rand(12, V, generator=g) < 0.05).to(torch.int32).to(DEV)
    routes = [dict(top_k=0, top_p=1.0, min_p=0.0, rep=1.0), dict(top_k=20, top_p=0.9, min_p=0.0, rep=1.1),
              dict(top_k=min(2000, V - 1), top_p=0.7, min_p=0.0, rep=1.0), dict(top_k=0, top_p=0.9, min_p=0.01, rep=1.2)]

    def draw(rows_total, route):
        reps = -(-rows_total // 12)
        logits = base.repeat(reps, 1)[:rows_total].contiguous()
        counts = counts_base.repeat(reps, 1)[:rows_total].contiguous()
        n = rows_total
        f = lambda v: torch.full((n,), v, dtype=torch.float32, device=DEV)
        idx = torch.arange(n, dtype=torch.int32, device=DEV)
        out = ops.sample(logits, temperature=f(0.9), seeds=(idx % 12).to(torch.int64) + 100, draw_index=(idx % 12) * 3,
                         top_k=torch.full((n,), route["top_k"], dtype=torch.int32, device=DEV), top_p=f(route["top_p"]),
                         min_p=f(route["min_p"]), repetition_penalty=f(route["rep"]), presence_penalty=f(0.1),
                         frequency_penalty=f(0.05), count_rows=idx, counts=counts)
        return out.cpu().numpy()

    for route in routes:
        alone = draw(12, route)                 # 8 CTAs a row
        assert draw(1, route)[0] == alone[0]
        for n in (30, 70, 200):                 # 4, 2 and 1 CTAs a row
            got = draw(n, route)
            assert (got == np.resize(alone, n)).all(), f"{route}: a draw changed with {n} rows in the launch"
        assert len(set(alone.tolist())) > 3


def test_greedy_rows_penalties_and_counts():
    from zinfer_b200 import ops

    V = 301
    logits = torch.zeros(3, V, device=DEV)
    logits[:, 7] = 3.0
    logits[:, 9] = 2.9
    counts = torch.zeros(2, V, dtype=torch.int32, device=DEV)
    ops.count_tokens(counts[1], torch.tensor([7, 7, 3], dtype=torch.int32, device=DEV))
    assert counts[1, 7] == 2 and counts[1, 3] == 1
    f = lambda *v: torch.tensor(v, dtype=torch.float32, device=DEV)
    i = lambda *v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = ops.sample(logits, temperature=f(0.0, 0.0, 1.0), seeds=torch.zeros(3, dtype=torch.int64, device=DEV),
                     draw_index=i(0, 0, 0), top_k=i(0, 0, 1), top_p=f(1, 1, 1), min_p=f(0, 0, 0),
                     repetition_penalty=f(1, 1, 1), presence_penalty=f(0, 0.2, 0), frequency_penalty=f(0, 0, 0),
                     count_rows=i(-1, 1, 0), counts=counts)
    # row 0: plain argmax; row 1: token 7 was seen, its logit drops by 0.2 below token 9; row 2: top_k = 1 is greedy
    assert out.tolist() == [7, 9, 7]
    assert counts[1, 9] == 1 and counts[0, 7] == 1   # the drawn tokens were counted


def test_temperature_generation_is_reproducible_and_independent_of_batching(model_dirs):
    from zinfer_b200.sampling import SamplingParams

    d = model_dirs[("B", "float32")]
    prompts = [[3], list(range(1, 10)), list(range(5, 45)), list(range(100, 170))]
    sp = SamplingParams(temperature=0.8, seed=42, max_new_tokens=24, ignore_eos=True)
    together = _engine(d, "B", "float32").generate(prompts, sp)
    alone = [_engine(d, "B", "float32", max_batched_tokens=64).generate([p], sp)[0] for p in prompts]
    assert [r.token_ids for r in together] == [r.token_ids for r in alone]
    assert len({tuple(r.token_ids) for r in together}) == 4
    other = _engine(d, "B", "float32").generate(prompts, SamplingParams(temperature=0.8, seed=43, max_new_tokens=24, ignore_eos=True))
    assert [r.token_ids for r in other] != [r.token_ids for r in together]
