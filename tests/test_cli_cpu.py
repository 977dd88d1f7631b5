"""The command line's parsing and its inspection commands (no GPU), and generation
through the Python entry point with the kernels replaced by their references."""
import io

import pytest
import torch

import plain_qwen3
from conftest import PAGE_SIZE
from zinfer_b200 import cli


def test_token_id_csv():
    assert cli.parse_token_ids("1, 2,3") == [1, 2, 3]
    with pytest.raises(cli.CliError, match="InvalidTokenId"):
        cli.parse_token_ids("1,x")


def test_flags_have_the_reference_names_and_errors():
    s, e = cli.parse_flags(["--seed", "7", "--temperature", "0.6", "--top-p", "0.95", "--top-k", "20", "--min-p", "0.1",
                            "--presence-penalty", "0.5", "--frequency-penalty", "0.2", "--repetition-penalty", "1.1",
                            "--dtype", "float32", "--chunk-size", "16", "--ignore-eos"])
    assert s == dict(seed=7, temperature=0.6, top_p=0.95, top_k=20, min_p=0.1, presence_penalty=0.5,
                     frequency_penalty=0.2, repetition_penalty=1.1, ignore_eos=True)
    assert e == dict(dtype="float32", chunk_size=16)
    with pytest.raises(cli.CliError, match="MissingFlagValue"):
        cli.parse_flags(["--seed"])
    with pytest.raises(cli.CliError, match="UnknownFlag"):
        cli.parse_flags(["--threads", "3"])


def test_inspect_commands(model_dirs):
    d = model_dirs[("B", "bfloat16")]
    out = io.StringIO()
    assert cli.run(["inspect-config", d], out) == 0
    text = out.getvalue()
    assert "Zinfer model inspection" in text and "num_key_value_heads: 1" in text and "head_dim: 32" in text
    out = io.StringIO()
    assert cli.run(["inspect-weights", d], out) == 0
    assert "tensor_count: 36" in out.getvalue()
    out = io.StringIO()
    assert cli.run(["inspect-tensor", d, "model.norm.weight", "3"], out) == 0
    assert out.getvalue().count("value[") == 3
    assert cli.run(["inspect-tensor", d, "nope"], io.StringIO()) == 2
    assert cli.run(["frobnicate"], io.StringIO()) == 2
    assert cli.run(["inspect-config", "/nonexistent"], io.StringIO()) == 1


def test_random_model_command(tmp_path, model_dirs):
    import os
    out = io.StringIO()
    cfg = os.path.join(model_dirs[("A", "bfloat16")], "config.json")
    assert cli.run(["random-model", str(tmp_path / "m"), cfg, "9"], out) == 0
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]


@pytest.mark.parametrize("name", ["A", "B"])
def test_generate_matches_plain_greedy_on_cpu(cpu_kernels, model_dirs, name):
    from zinfer_b200.engine.api import Engine
    from zinfer_b200.sampling import SamplingParams

    d = model_dirs[(name, "float32")]
    cfg, w = plain_qwen3.load_model(d)
    prompts = [[3, 9, 27, 81, 5], [7] * 17, list(range(1, 34))]
    eng = Engine(d, dtype="float32", device="cpu", page_size=PAGE_SIZE[name], kv_cache_tokens=512,
                 max_batched_tokens=16, max_requests=4)
    res = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True))
    for p, r in zip(prompts, res):
        assert r.token_ids == plain_qwen3.greedy(cfg, w, p, 6) and r.finish_reason == "length"
    # so few pages that requests are preempted and recomputed: the tokens stay the same
    ps = PAGE_SIZE[name]
    prompts = [[(7 * i + j) % 200 + 1 for j in range(ps - 1 - i)] for i in range(3)]
    want = [plain_qwen3.greedy(cfg, w, p, 6) for p in prompts]
    tight = Engine(d, dtype="float32", device="cpu", page_size=ps, num_pages=4, max_batched_tokens=16, max_requests=4)
    res2 = tight.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True))
    assert [r.token_ids for r in res2] == want
    assert tight.scheduler.stats.preemptions > 0 and res2[0].preemptions == 0
    tight.runner.manager.check()
    assert not tight.runner.manager.requests
