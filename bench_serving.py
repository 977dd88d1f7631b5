#!/usr/bin/env python3
"""Continuous-batching workloads on one B200, through the public Engine.

    python bench_serving.py --workload 14b    # Qwen3-14B shape: 32 requests, prompts U[128, 3072],
                                              # chunked prefill of 512 mixed with decode, 128 greedy tokens each
    python bench_serving.py --workload 32b    # Qwen3-32B shape: 16 requests of 4,096 prompt + 512 tokens at
                                              # temperature 0.7, the paged cache sized just above what they hold

Random bfloat16 weights, seeded uniform-random token ids.  Prints key: value lines in the
reference's manner (src/app/cli/tools/bench/runtime.zig:284-309) and one JSON line.
"""
import argparse
import json
import random
import sys
import time

import torch

from zinfer_b200.config import Qwen3Config
from zinfer_b200.engine.api import Engine
from zinfer_b200.sampling import SamplingParams

SHAPES = {
    "14b": dict(num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                intermediate_size=17408, context=4096),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                intermediate_size=25600, context=8192),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=sorted(SHAPES), default="14b")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers (reported)")
    ap.add_argument("--requests", type=int, default=None)
    args = ap.parse_args()
    shape = dict(SHAPES[args.workload])
    context = shape.pop("context")
    full_layers = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    cfg = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, max_position_embeddings=40960,
        rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, torch_dtype="bfloat16", **shape))
    rng = random.Random(7)
    if args.workload == "14b":
        n = args.requests or 32
        prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(128, 3072))] for _ in range(n)]
        params = SamplingParams(temperature=0.0, max_new_tokens=128, ignore_eos=True)
        opts = dict(max_batched_tokens=512, chunk_size=512, max_requests=n, kv_cache_tokens=n * 3200 + 1024)
    else:
        n = args.requests or 16
        prompts = [[rng.randrange(cfg.vocab_size) for _ in range(4096)] for _ in range(n)]
        params = SamplingParams(temperature=0.7, seed=11, max_new_tokens=512, ignore_eos=True)
        opts = dict(max_batched_tokens=2048, chunk_size=2048, max_requests=n, kv_cache_tokens=n * (4096 + 512) + 256)
    t0 = time.perf_counter()
    engine = Engine(config=cfg, random_weights_seed=3, dtype="bfloat16", max_model_len=context, page_size=16, **opts)
    torch.cuda.synchronize()
    load_s = time.perf_counter() - t0
    engine.generate([prompts[0][:64]], SamplingParams(temperature=0.0, max_new_tokens=4, ignore_eos=True))   # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    results = engine.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = engine.scheduler.stats
    prompt_tokens = sum(len(p) for p in prompts)
    decoded = sum(len(r.token_ids) for r in results)
    out = {
        "workload": args.workload, "layers": cfg.num_hidden_layers, "layers_full_model": full_layers, "requests": n,
        "prompt_tokens": prompt_tokens, "decoded_tokens": decoded, "seconds": round(dt, 3),
        "total_tok_s": round((prompt_tokens + decoded) / dt, 1), "decode_tok_s": round(decoded / dt, 1),
        "steps": st.steps, "preemptions": st.preemptions, "finish_reasons": sorted({r.finish_reason for r in results}),
        "weights_gb": round(engine.runner.model.weight_bytes() / 1e9, 2),
        "kv_cache_gb": round(engine.runner.storage.bytes() / 1e9, 2), "load_seconds": round(load_s, 1),
    }
    for k, v in out.items():
        print(f"{k}: {v}")
    print(json.dumps(out))
    engine.runner.manager.check()
    return 0


if __name__ == "__main__":
    sys.exit(main())
