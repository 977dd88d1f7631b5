"""The engine against the plain model at the benchmark's layer sizes.

Every other comparison with the plain model runs at widths up to 320.  This one uses
the layer sizes that bench.py times (Qwen3-8B: width 4096, 32 query and 8 kv heads of
128, feed-forward 12288, vocabulary 151,936, separate output head) with 2 of the 36
layers, so that what is compared is what is timed: the tcgen05 products with their
K splits at K = 4096 and 12288, the tcgen05 prefill attention, the fused decode
attention under CUDA graphs, the unfused decode route that 64 requests take, and the
output head over the whole vocabulary.  The plain model runs the same bfloat16 weight
values in float64 (on the GPU through plain torch operations: 1.3 billion parameters
are too slow for the CPU in a test; it shares no code with the engine either way).
"""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as ru

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LAYERS, LAYERS_FULL_MODEL = 2, 36
SHAPE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
    intermediate_size=12288, num_hidden_layers=LAYERS, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
    torch_dtype="bfloat16")
# Measured on a B200 (worst of all compared rows, as a fraction of the row's largest logit, each row
# being the worst of 151,936 logits): bfloat16 tail 1.15e-2, mixed 1.11e-2, 64 requests 1.22e-2;
# float32 whole 6.0e-6.  The limits are twice the largest of these.
TOL = {"bfloat16": dict(rtol=2.5e-2, atol=1e-3), "float32": dict(rtol=1.2e-5, atol=1e-6)}


@pytest.fixture(scope="module")
def shape_model():
    """(config dict, bfloat16 tensors by name on the device, the same values in float64 for the plain model)."""
    from zinfer_b200.config import Qwen3Config
    from zinfer_b200.config.qwen3 import qwen3_model_spec
    from zinfer_b200.engine.model import declared_tensors
    from zinfer_b200.weights import random_tensors

    cfg = Qwen3Config.from_dict(SHAPE)
    specs = {n: s for n, s in declared_tensors(qwen3_model_spec(cfg)).items() if not s.optional}
    tensors = random_tensors(specs, 808, torch.bfloat16, DEV)
    plain_w = {n: t.to(torch.float64) for n, t in tensors.items()}
    yield cfg, tensors, plain_w
    del tensors, plain_w
    torch.cuda.empty_cache()


def _runner(cfg, tensors, dtype, **kw):
    from zinfer_b200.config.qwen3 import qwen3_model_spec
    from zinfer_b200.engine import DecoderModel, ModelRunner

    model = DecoderModel(qwen3_model_spec(cfg), dtype, DEV)
    model.bind({n: t.to(dtype) for n, t in tensors.items()})
    return ModelRunner(model, page_size=16, **kw)


def _plain_rows(plain_w, reqs, results):
    """{request: {position: logits row}} of the plain model at the positions that were returned."""
    out = {}
    for rid, toks in reqs.items():
        rows = sorted(pos for (r, pos) in results if r == rid)
        if rows:
            logits = P.forward(SHAPE, plain_w, toks, rows=rows).cpu().numpy()
            out[rid] = {pos: logits[i] for i, pos in enumerate(rows)}
    return out


def _compare(results, plain_w, reqs, dtype, what):
    worst = ru.assert_close(results, _plain_rows(plain_w, reqs, results), what=what, argmax_frac=0.9, **TOL[dtype])
    print(f"measured {what}: worst error {worst * TOL[dtype]['rtol']:.2e} of the row's largest logit, {len(results)} rows")


def test_prompt_in_one_step_then_the_tail_token_by_token(shape_model):
    """A prompt of 330 tokens in one step (token-major tcgen05 products, tcgen05 prefill attention),
    then 32 single tokens: the first uncaptured, the rest replayed from the CUDA graph of (1 request, 384 keys)
    with the fused decode attention and K-split products."""
    cfg, tensors, plain_w = shape_model
    runner = _runner(cfg, tensors, torch.bfloat16, max_tokens=512, max_requests=4)
    reqs = ru.make_requests(cfg.vocab_size, [362], seed=5)
    trace = ru.trace_tail_decode(reqs, 32)
    trace[0]["entries"][0]["want"] = [0, 1, 127, 128, 200, 329]
    got = ru.run_in_process(runner, trace)
    assert runner.graphs is not None and runner.graphs.replays >= 30, "the single tokens did not run from a CUDA graph"
    _compare(got, plain_w, reqs, "bfloat16", "8B shape / bfloat16 / tail")


def test_four_live_requests_in_a_small_pool(shape_model):
    """Portions of some requests beside decoded tokens of others, up to four live, pages used again."""
    cfg, tensors, plain_w = shape_model
    reqs = ru.make_requests(cfg.vocab_size, [150, 90, 260, 60, 131, 17], seed=6)
    trace = ru.trace_mixed(reqs, 13)
    runner = _runner(cfg, tensors, torch.bfloat16, max_tokens=ru.max_live_tokens(trace), max_requests=4)
    got = ru.run_in_process(runner, trace)
    assert runner.manager.groups[0].pool.reused > 0, "no page was used again"
    _compare(got, plain_w, reqs, "bfloat16", "8B shape / bfloat16 / mixed")


def test_sixty_four_requests_decode_together(shape_model):
    """64 requests take the decode attention's separate kernels (64 x 8 kv heads are more blocks than
    fit at once, so the fused form is not used) and the 64-token products; three steps: uncaptured,
    captured, replayed."""
    from zinfer_b200 import ops

    cfg, tensors, plain_w = shape_model
    assert 64 * cfg.num_key_value_heads > 2 * torch.cuda.get_device_properties(0).multi_processor_count
    runner = _runner(cfg, tensors, torch.bfloat16, max_tokens=64 * 64, max_requests=64)
    reqs = ru.make_requests(cfg.vocab_size, [20 + (i * 7) % 23 for i in range(64)], seed=7)
    ids = list(reqs)
    trace = []
    for i in range(0, 64, 16):      # prompts without their last three tokens, 16 requests a step
        trace.append({"step": len(trace), "end": [],
                      "entries": [{"id": r, "tokens": reqs[r][:-3], "want": []} for r in ids[i:i + 16]]})
    for k in (3, 2, 1):
        trace.append({"step": len(trace), "end": ids if k == 1 else [],
                      "entries": [{"id": r, "tokens": reqs[r][-k:len(reqs[r]) - k + 1], "want": [0]} for r in ids]})
    got = ru.run_in_process(runner, trace)
    assert runner.graphs.replays >= 2 and len(got) == 3 * 64
    _compare(got, plain_w, reqs, "bfloat16", "8B shape / bfloat16 / 64 requests")
    ops.require_kernel_status_ok("8B shape")


@pytest.mark.parametrize("n", [3, 64])
def test_greedy_ids_from_the_heads_epilogue(shape_model, n):
    """Greedy decoding takes the row maxima that the output head's product leaves per 32 weight rows
    (151,936 weight rows: 4,748 candidates a token): the ids are the first maxima of the logits
    returned beside them, and the logits are those of the plain step; uncaptured, captured, replayed."""
    from zinfer_b200.engine import StepEntry

    cfg, tensors, _ = shape_model
    runner = _runner(cfg, tensors, torch.bfloat16, max_tokens=n * 64, max_requests=n)
    twin = _runner(cfg, tensors, torch.bfloat16, max_tokens=n * 64, max_requests=n)
    reqs = ru.make_requests(cfg.vocab_size, [9 + (i * 5) % 17 for i in range(n)], seed=11)
    for r in (runner, twin):
        for rid, toks in reqs.items():
            r.add_request(rid)
        r.step([StepEntry(rid, toks[:-1], []) for rid, toks in reqs.items()])
    cur = [toks[-1] for toks in reqs.values()]
    for _ in range(3):
        entries = [StepEntry(rid, [t], [0]) for rid, t in zip(reqs, cur)]
        logits, ids = runner.step_argmax(entries)
        assert ids.dtype == torch.int32 and torch.equal(ids.long(), torch.argmax(logits, dim=-1))
        assert torch.equal(logits, twin.step(entries))
        cur = ids.tolist()
    assert runner.graphs.replays >= 1


def test_float32_whole_prompts(shape_model):
    """The true 32-bit path at these sizes: CUDA-core products over K = 12288 and the exact attention."""
    cfg, tensors, plain_w = shape_model
    runner = _runner(cfg, tensors, torch.float32, max_tokens=256, max_requests=2)
    reqs = ru.make_requests(cfg.vocab_size, [70, 33], seed=8)
    trace = ru.trace_whole(reqs)
    for st in trace:
        st["entries"][0]["want"] = st["entries"][0]["want"][::7]
    got = ru.run_in_process(runner, trace)
    _compare(got, plain_w, reqs, "float32", "8B shape / float32 / whole")
