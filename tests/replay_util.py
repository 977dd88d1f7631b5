"""Traces for replay tests: the same requests whole, with the tail decoded one by
one, in portions of changing size, and mixed with other requests; helpers to run
a trace in process or through bin/trace_run and to compare with the plain model."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_requests(vocab: int, lengths, seed: int) -> dict[str, list[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


# ------------------------------------------------------------------------ traces
def trace_whole(reqs) -> list[dict]:
    """Each request alone and whole: one step, every position wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(reqs.items())]


def trace_tail_decode(reqs, tail: int = 32) -> list[dict]:
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[p:p + 1], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(reqs, seed: int, sizes=(7, 2, 13, 2, 5, 3, 31, 2, 16, 17, 1, 64)) -> list[dict]:
    """Portions of changing size, down to two tokens (and one)."""
    rng = random.Random(seed)
    steps = []
    for rid, toks in reqs.items():
        p, k = 0, rng.randrange(len(sizes))
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}],
                          "end": [rid] if p + n == len(toks) else []})
            p += n
    return steps


def trace_mixed(reqs, seed: int, max_live: int = 4, tail: int = 12) -> list[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens
    of others in one step; some requests sit a step out; finished requests' pages
    go to the ones that start later."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: dict[str, int] = {}   # id -> tokens fed so far
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            toks, p = reqs[rid], live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # this request is left out of the step
            left = len(toks) - p
            if left <= tail:
                n = 1
            else:
                n = min(left - tail, rng.choice([2, 2, 3, 5, 8, 13, 21, 40]))
            want = list(range(n)) if n <= 4 or rng.random() < 0.5 else sorted(rng.sample(range(n), 3))
            entries.append({"id": rid, "tokens": toks[p:p + n], "want": want})
            live[rid] = p + n
            if p + n == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            rng.shuffle(entries)
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(trace, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for st in trace:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


# ----------------------------------------------------------------------- running
def collect(trace, logits_of_step) -> dict[tuple[str, int], np.ndarray]:
    """{(request, position): logits row} from per-step logit arrays."""
    fed: dict[str, int] = {}
    out = {}
    for st in trace:
        arr = logits_of_step(st["step"])
        row = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = arr[row]
                row += 1
            fed[e["id"]] = base + len(e["tokens"])
        assert arr is None or row == len(arr), "the step wrote a different number of rows than were wanted"
    return out


def run_in_process(runner, trace):
    from zinfer_b200.engine import StepEntry

    results = {}
    for st in trace:
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]])
        results[st["step"]] = None if logits is None else logits.float().cpu().numpy()
        for rid in st["end"]:
            runner.end_request(rid)
    runner.manager.check()
    return collect(trace, lambda s: results[s])


def run_trace_tool(model_dir: str, dtype: str, trace, out_dir: str, max_tokens: int, vocab: int, extra=(), info=None):
    """Runs bin/trace_run as a user would and reads back what it wrote.  ``info`` (a dict)
    receives ``pages_reused``: how many page allocations returned a page that had been used before."""
    cmd = [sys.executable, os.path.join(REPO, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), *extra]
    inp = "".join(json.dumps(st) + "\n" for st in trace)
    r = subprocess.run(cmd, input=inp, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [ln for ln in r.stdout.splitlines() if ln.startswith("done ")]
    assert [ln.split()[1] for ln in done] == [str(st["step"]) for st in trace], "trace_run did not confirm every step"
    if info is not None:
        import re
        m = re.search(r"(\d+) page allocations returned a page used before", r.stderr)
        info["pages_reused"] = int(m.group(1)) if m else None

    def load(step):
        path = os.path.join(out_dir, f"{step}.f32")
        if not os.path.exists(path):
            return None
        return np.fromfile(path, dtype="<f4").reshape(-1, vocab)

    return collect(trace, load)


# --------------------------------------------------------------------- comparing
def plain_logits(cfg: dict, weights, reqs) -> dict[str, np.ndarray]:
    import plain_qwen3

    return {rid: plain_qwen3.forward(cfg, weights, toks).numpy() for rid, toks in reqs.items()}


def assert_close(results, plain, rtol: float, atol: float, argmax_frac: float = 1.0, what: str = "") -> float:
    """Every returned row against the plain model's row at the same position.  The
    error is measured against the largest logit of that row, so it means the same
    for every model size.  Beyond the fraction ``argmax_frac`` of rows whose best token
    must agree outright, the best token must agree on EVERY row where the plain model's
    lead of the best over the second best is more than twice the tolerance (two logits
    that each move by the tolerance cannot change places then).  Returns the worst
    error as a fraction of the tolerance."""
    assert results, "nothing to compare"
    worst, worst_key, agree = 0.0, None, 0
    for (rid, pos), row in sorted(results.items()):
        ref = np.asarray(plain[rid][pos])
        assert np.isfinite(row).all(), f"{what}: non-finite logits at {rid}[{pos}]"
        lim = atol + rtol * np.abs(ref).max()
        err = np.abs(row.astype(np.float64) - ref).max() / lim if lim > 0 else 0
        if err > worst:
            worst, worst_key = err, (rid, pos)
        same = int(np.argmax(row)) == int(np.argmax(ref))
        agree += int(same)
        if not same:
            top2 = np.partition(ref, -2)[-2:]
            assert top2[1] - top2[0] <= 2 * lim, (f"{what}: at {rid}[{pos}] the plain model prefers token {int(np.argmax(ref))} "
                                                  f"by {top2[1] - top2[0]:.3g} (tolerance {lim:.3g}), the engine chose {int(np.argmax(row))}")
    assert worst <= 1.0, (f"{what}: logits differ from the plain model by {worst:.2f}x the tolerance "
                          f"(rtol={rtol}, atol={atol}); first look at {worst_key}: {first_bad(results, plain, rtol, atol)}")
    assert agree >= argmax_frac * len(results), f"{what}: argmax agrees on only {agree} of {len(results)} rows"
    return worst


def first_bad(results, plain, rtol, atol):
    for (rid, pos), row in sorted(results.items()):
        ref = plain[rid][pos]
        if np.abs(row.astype(np.float64) - ref).max() > atol + rtol * np.abs(ref).max():
            return f"first wrong place in order: request {rid}, position {pos}"
    return "none"
