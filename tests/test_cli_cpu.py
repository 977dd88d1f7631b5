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


def test_engine_and_run_flags():
    run = {}
    s, e = cli.parse_flags(["--num-pages", "12", "--kv-cache-bytes", "1000000", "--gpu-memory-fraction", "0.5",
                            "--max-model-len", "99", "--max-requests", "3", "--random-weights", "7", "--config", "c.json",
                            "--max-new-tokens", "5", "--profile", "p.json"], run)
    assert s == {} and e == dict(num_pages=12, kv_cache_bytes=1000000, gpu_memory_fraction=0.5, max_model_len=99, max_requests=3)
    assert run == dict(random_weights=7, config="c.json", max_new_tokens=5, profile="p.json")
    with pytest.raises(cli.CliError, match="go together"):
        cli.ModelSource("x", {"random_weights": 1})


def test_generate_several_prompts_from_random_weights_without_a_folder(cpu_kernels, model_dirs, tmp_path):
    import os

    cfg_path = os.path.join(model_dirs[("A", "float32")], "config.json")
    common = ["--random-weights", "11", "--config", cfg_path, "--device", "cpu", "--dtype", "float32", "--ignore-eos",
              "--temperature", "0"]
    out = io.StringIO()
    assert cli.run(["generate", "1,2,3;4,5;9", "--max-new-tokens", "4", *common], out) == 0
    lines = out.getvalue().splitlines()
    toks = [ln for ln in lines if ln.startswith("tokens[")]
    assert len(toks) == 3 and all(ln.count(",") == 3 for ln in toks)
    assert sum(ln.startswith("finish_reason[") and ln.endswith("length") for ln in lines) == 3
    # each prompt alone, positional max_new_tokens: the same tokens
    for i, p in enumerate(("1,2,3", "4,5", "9")):
        alone = io.StringIO()
        assert cli.run(["generate", p, "4", *common], alone) == 0
        assert alone.getvalue().splitlines()[0].split(": ")[1] == toks[i].split(": ")[1]
    # random-model writes a sharded folder, which the commands read like any other
    assert cli.run(["random-model", str(tmp_path / "m"), cfg_path, "11", "--shards", "2"], io.StringIO()) == 0
    folder = io.StringIO()
    assert cli.run(["generate", str(tmp_path / "m"), "1,2,3", "4", "--device", "cpu", "--dtype", "float32", "--ignore-eos",
                    "--temperature", "0"], folder) == 0
    assert folder.getvalue().startswith("tokens: [")
    out = io.StringIO()
    assert cli.run(["inspect-weights", str(tmp_path / "m")], out) == 0
    assert "shard_count: 2" in out.getvalue()
    assert cli.run(["generate", "1,2", "--random-weights", "1"], io.StringIO()) == 2


def test_pool_sizing_from_a_byte_budget(cpu_kernels, model_dirs):
    from zinfer_b200.cache import bytes_per_page, bytes_per_token, pages_for
    from zinfer_b200.engine.api import Engine
    from zinfer_b200.parts import KVCacheNeed

    needs = {"a": KVCacheNeed(2, 16, None), "b": KVCacheNeed(2, 16, None), "c": KVCacheNeed(1, 32, 64)}
    # two caches share a group; the third has its own: one page id costs a page in each
    assert bytes_per_page(needs, 16, 2) == (2 * 2 * 2 * 16 * 16 + 1 * 2 * 1 * 16 * 32) * 2
    assert bytes_per_token(needs, 2) * 16 == bytes_per_page(needs, 16, 2)
    per = bytes_per_page(needs, 16, 2)
    assert pages_for(needs, 16, 2, budget_bytes=10 * per + per - 1) == 10
    assert pages_for(needs, 16, 2, budget_bytes=10 * per, tokens=33) == 3       # capped by what the tokens need
    assert pages_for(needs, 16, 2, budget_bytes=0) == 1
    # Tiny A: 2 layers x 2 kv heads x 16 x 4 bytes x 2 = 512 bytes a token in float32
    eng = Engine(model_dirs[("A", "float32")], dtype="float32", device="cpu", page_size=16, kv_cache_bytes=512 * 16 * 7 + 100,
                 max_requests=4)
    assert eng.runner.manager.groups[0].pool.num_pages == 7
    assert eng.runner.storage.bytes() == 512 * 16 * 7
    # the default: as many tokens as the requests could fill, where no device memory can be asked
    eng = Engine(model_dirs[("A", "float32")], dtype="float32", device="cpu", page_size=16, max_requests=4)
    assert eng.runner.manager.groups[0].pool.num_pages == 4 * 128 // 16


def test_stop_and_stream_flags(cpu_kernels, model_dirs):
    """--stop (repeatable, ids for the reference's text) and --stream through the command line."""
    run = {}
    s, _ = cli.parse_flags(["--stop", "5,6", "--stop", "7", "--stream"], run)
    assert s == dict(stop_sequences=[[5, 6], [7]]) and run == dict(stream=True)
    with pytest.raises(cli.CliError, match="MissingFlagValue"):
        cli.parse_flags(["--stop"], {})
    d = model_dirs[("A", "float32")]
    cfg, w = plain_qwen3.load_model(d)
    full = plain_qwen3.greedy(cfg, w, [3, 9, 27], 8)
    stop = ",".join(map(str, full[4:6]))
    cut = next(i for i in range(7) if full[i:i + 2] == full[4:6])
    out = io.StringIO()
    assert cli.run(["generate", d, "3,9,27", "8", "--device", "cpu", "--dtype", "float32", "--temperature", "0", "--ignore-eos",
                    "--stop", stop, "--stream"], out) == 0
    text = out.getvalue()
    streamed = [int(t) for line in text.splitlines() if line.startswith("stream[0]: ") for t in line.split(": ")[1].split()]
    assert streamed == full[:cut]
    assert "tokens: [" + ", ".join(map(str, full[:cut])) + "]" in text and "finish_reason: stop" in text
