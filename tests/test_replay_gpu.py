"""Trace replay on the GPU through bin/trace_run, as a user runs it: the same
requests whole, with the tail decoded token by token, in portions of changing
size, and mixed with other requests in a pool so small that pages are reused; in
float32 and in bfloat16; every wanted row against the plain model."""
import pytest

import plain_qwen3
import replay_util as ru

pytestmark = pytest.mark.gpu

# float32: both sides round every operation to 24 bits and the plain model runs in
# float64, so rows agree to a few 1e-6 of the row's largest logit; 5e-5 leaves room
# for the longer sums of the larger shapes.  bfloat16: activations are rounded to 8
# bits between kernels (2^-9 relative each), which accumulates over a few layers.
# MEASURED holds the worst error seen on a B200 per configuration (as a fraction of the
# row's largest logit, over all four ways of cutting); the bfloat16 limit is twice that.
# Beyond the limits, the best token must agree wherever the plain model's lead exceeds
# twice the tolerance (replay_util.assert_close).
MEASURED_BF16 = {"A": 6.8e-3, "B": 8.4e-3, "C": 6.7e-3, "D": 1.05e-2, "E": 8.3e-3}
TOL = {"float32": lambda name: dict(rtol=5e-5, atol=1e-6),
       "bfloat16": lambda name: dict(rtol=2 * MEASURED_BF16[name], atol=1e-3)}
LENGTHS = {"A": [5, 17, 33, 64, 100], "B": [1, 9, 40, 70, 129, 200], "C": [3, 77, 150, 31],
           "D": [2, 65, 130, 300, 47], "E": [1, 129, 64, 200]}


def _trace(mode, reqs):
    return {"whole": lambda: ru.trace_whole(reqs), "tail": lambda: ru.trace_tail_decode(reqs, 32),
            "portions": lambda: ru.trace_portions(reqs, 11), "mixed": lambda: ru.trace_mixed(reqs, 13)}[mode]()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_every_way_of_cutting(model_dirs, tmp_path, name, dtype):
    from conftest import PAGE_SIZE

    model_dir = model_dirs[(name, dtype)]
    cfg, w = plain_qwen3.load_model(model_dir)
    reqs = ru.make_requests(cfg["vocab_size"], LENGTHS[name], seed=21)
    plain = ru.plain_logits(cfg, w, reqs)
    results, worst = {}, 0.0
    for mode in ("whole", "tail", "portions", "mixed"):
        trace = _trace(mode, reqs)
        out = tmp_path / mode
        info = {}
        # in the mixed run every page is overwritten with huge values when it is given back: what a
        # page held before must not reach any result
        extra = ["--page-size", str(PAGE_SIZE[name])] + (["--poison-freed-pages"] if mode == "mixed" else [])
        results[mode] = ru.run_trace_tool(model_dir, dtype, trace, str(out), ru.max_live_tokens(trace),
                                          cfg["vocab_size"], extra=extra, info=info)
        if mode == "mixed":
            assert info["pages_reused"], "the mixed trace is meant to use pages again, and did not"
        tol = TOL[dtype](name)
        worst = max(worst, tol["rtol"] * ru.assert_close(results[mode], plain, what=f"{name}/{dtype}/{mode}", **tol,
                                                         argmax_frac=1.0 if dtype == "float32" else 0.8))
    print(f"measured {name}/{dtype}: worst error {worst:.2e} of the row's largest logit")
    # the ways of cutting agree with each other far more closely than with the plain model
    for mode in ("tail", "portions", "mixed"):
        for key, row in results[mode].items():
            ref = results["whole"][key]
            scale = abs(ref).max()
            lim = 2e-5 * scale if dtype == "float32" else 2e-2 * scale
            assert abs(row - ref).max() <= lim, f"{name}/{dtype}: {mode} differs from whole at {key}"
