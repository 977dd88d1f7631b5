"""The engine's host logic (batching, block tables, cache reuse, step function)
without a GPU: the kernels are replaced by their plain PyTorch references
(tests/kernel_refs.py), everything else is the product's own code."""
import pytest
import torch

import plain_qwen3
import replay_util as ru
from conftest import PAGE_SIZE, TINY


def _runner(model_dirs, name, max_tokens):
    from zinfer_b200.engine import ModelRunner

    return ModelRunner.from_model_dir(model_dirs[(name, "float32")], dtype=torch.float32, device="cpu",
                                      page_size=PAGE_SIZE[name], max_tokens=max_tokens, max_requests=8)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_matches_plain_on_cpu(cpu_kernels, model_dirs, name, mode):
    cfg, w = plain_qwen3.load_model(model_dirs[(name, "float32")])
    lengths = [5, 17, 33, 40] if name == "A" else [1, 9, 40, 70, 23]
    reqs = ru.make_requests(cfg["vocab_size"], lengths, seed=7)
    trace = {"whole": ru.trace_whole(reqs), "tail": ru.trace_tail_decode(reqs, 12),
             "portions": ru.trace_portions(reqs, 3), "mixed": ru.trace_mixed(reqs, 5)}[mode]
    runner = _runner(model_dirs, name, ru.max_live_tokens(trace))
    got = ru.run_in_process(runner, trace)
    ru.assert_close(got, ru.plain_logits(cfg, w, reqs), rtol=2e-5, atol=1e-6, what=f"{name}/{mode}")
    assert not runner.manager.requests and all(g.pool.num_used == 0 for g in runner.manager.groups)
