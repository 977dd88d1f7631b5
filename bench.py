#!/usr/bin/env python3
"""Benchmark of the engine's decode step on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Default: the layer sizes of the Qwen3-8B shape, random bfloat16 weights, batch 8,
each request holding a 2,048-token prompt, engine context limit 4,096; token ids
are seeded uniform-random (no dataset).  A step is one decode step (one new token
for every request).  Prints ONE JSON line:

  value     decoded tokens per second at batch 8, timed on the device with CUDA events
  e2e       the same through the Python entry point (Engine.step), host tokens in
            and out, with the step's host->device and device->host bytes; "points"
            inside it: the same at batch 1 and 64; "sampled": the same at batch 8 with
            the reference's default sampling options instead of greedy
  prefill   one step of 2,048 prompt tokens: tokens/s, ms, fraction of the bf16 peak;
            "chunks_512" inside it: the same prompt as four steps of 512 tokens
  roofline  bytes the decode step must read (every weight once + the live
            requests' cache) / time, against the measured copy bandwidth
  points    decode tokens/s at batch 1 and 64

Peaks come from MEASURED_PEAKS.json when the driver wrote it, else the fallback
figures (6.65 TB/s, 1.59 PFLOP/s).  Weights (15 GB) exceed L2 (126 MB), so every
step streams its inputs from HBM without a flush.  For --gpus > 1 it says that
the engine is single-GPU and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
    intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
    torch_dtype="bfloat16")
PROMPT_LEN = 2048
CONTEXT_LEN = 4096
PREFILL_TOKENS = 2048


def peaks() -> tuple[float, float, str]:
    """(HBM GB/s, bf16 TFLOP/s, source)."""
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
        except (OSError, ValueError, KeyError):
            pass
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.rows: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()   # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def matmul_params(cfg, n_layers: int) -> int:
    """Weight elements every token multiplies with (layers + output head)."""
    H, I = cfg.hidden_size, cfg.intermediate_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = H * (q + 2 * kv) + q * H + 3 * H * I
    return n_layers * per_layer


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (reported in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="zinfer_b200", choices=["zinfer_b200", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (for profiling runs)")
    ap.add_argument("--profile", default=None, metavar="PATH",
                    help="also run one prefill and a few decode steps under the per-kernel-class profiler "
                         "(uncaptured, outside every timed region) and write its summary there as JSON")
    ap.add_argument("--timeline", default=None, metavar="PATH",
                    help="with ZINFER_B200_TRACE=1 in the environment: write the timeline of one decode step at the "
                         "headline batch (every kernel's start, the completion of what it depends on, and what it adds "
                         "to the chain) there as JSON, and do nothing else")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "NeoZedAtlas/Zinfer is a Zig program (needs zig >= 0.15.2); no Zig toolchain exists here and "
                          "pip cannot install it: it has neither setup.py nor pyproject.toml"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from zinfer_b200 import ops
    from zinfer_b200.config import Qwen3Config
    from zinfer_b200.engine import StepEntry
    from zinfer_b200.engine.api import Engine
    from zinfer_b200.sampling import SamplingParams

    full_layers = QWEN3_8B["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg = Qwen3Config.from_dict({**QWEN3_8B, "num_hidden_layers": n_layers})
    hbm_gbs, bf16_tflops, peak_src = peaks()
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(1234)
    max_batch = args.batch if args.skip_points else max(64, args.batch)
    steps, warmup = args.steps, args.warmup

    engine = Engine(config=cfg, random_weights_seed=20240, dtype="bfloat16", device="cuda:0", page_size=16,
                    kv_cache_tokens=max_batch * (PROMPT_LEN + steps + warmup + 64) + PREFILL_TOKENS + 64,
                    max_batched_tokens=max(PREFILL_TOKENS, 2048), max_requests=max_batch)
    runner = engine.runner
    weight_bytes = runner.model.weight_bytes() - cfg.vocab_size * cfg.hidden_size * 2   # the embedding table is only gathered
    kv_bytes_per_token = 2 * n_layers * cfg.num_key_value_heads * cfg.head_dim * 2

    def rand_tokens(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    def event_ms(fn, n):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(n):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end)

    if args.timeline:
        from zinfer_b200 import profiling

        ids = [f"t{i}" for i in range(args.batch)]
        for rid in ids:
            runner.step([StepEntry(rid, rand_tokens(PROMPT_LEN), [])])
        cur = torch.randint(0, cfg.vocab_size, (args.batch,), generator=gen).tolist()

        def one_step():
            runner.step_argmax([StepEntry(rid, [t], [0]) for rid, t in zip(ids, cur)])

        kernels = profiling.chain_timeline(one_step, warm=4)
        # the chain of a decode step of this architecture, when its kernel count says that it is the one meant
        per_layer = ["input norm", "qkv product", "attention (fused)", "attention combine", "o product", "post-attention norm",
                     "gate_up product", "swiglu", "down product"]
        names = ["embedding"] + per_layer * n_layers + ["final norm", "output head", "argmax (candidates)"]
        for i, k in enumerate(kernels):
            k["kernel"] = names[i] if len(names) == len(kernels) else f"kernel {i}"
        with open(args.timeline, "w") as f:
            json.dump({"batch": args.batch, "context": PROMPT_LEN, "layers": n_layers, "kernels": kernels}, f, indent=1)
        per = {}
        for k in kernels:
            if k["own_us"] is not None:
                per.setdefault(k["kernel"], []).append(k["own_us"])
        for name, v in per.items():
            print(f"{name:24s} {statistics.median(v):8.2f} us (median of {len(v)})")
        return 0

    # ---------------------------------------------------------------- prefill
    def prefill_once():
        runner.step([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])])
        runner.end_request("prefill")

    prompt = rand_tokens(PREFILL_TOKENS)
    for _ in range(2):
        prefill_once()
    pf_ms = event_ms(prefill_once, 3) / 3
    attn_flops = n_layers * 4 * cfg.num_attention_heads * cfg.head_dim * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2)
    pf_flops = 2 * PREFILL_TOKENS * matmul_params(cfg, n_layers) + attn_flops + 2 * cfg.vocab_size * cfg.hidden_size
    prefill = {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
               "frac": round(pf_flops / (pf_ms * 1e-3) / (bf16_tflops * 1e12), 4)}

    def prefill_chunked():
        for c in range(0, PREFILL_TOKENS, 512):
            last = c + 512 >= PREFILL_TOKENS
            runner.step([StepEntry("prefill", prompt[c:c + 512], [511] if last else [])])
        runner.end_request("prefill")

    prefill_chunked()
    ck_ms = event_ms(prefill_chunked, 3) / 3
    prefill["chunks_512"] = {"value": round(PREFILL_TOKENS / (ck_ms * 1e-3), 1), "ms": round(ck_ms, 3),
                             "frac": round(pf_flops / (ck_ms * 1e-3) / (bf16_tflops * 1e12), 4)}

    # ----------------------------------------------------------------- decode
    def decode_point(batch: int, n_steps: int, sample_clocks: bool = False):
        """Device-timed decode at `batch`: every request holds PROMPT_LEN cached tokens
        (their cache is filled by real prefill steps), then n_steps steps of one token each."""
        ids = [f"d{batch}_{i}" for i in range(batch)]
        for rid in ids:
            runner.step([StepEntry(rid, rand_tokens(PROMPT_LEN), [])])
        cur = torch.randint(0, cfg.vocab_size, (batch,), generator=gen).tolist()

        def one():
            nonlocal cur
            return runner.step_argmax([StepEntry(rid, [t], [0]) for rid, t in zip(ids, cur)])[1]

        for _ in range(warmup):
            one()
        launches0 = ops.LAUNCHES + runner.graph_launches if hasattr(runner, "graph_launches") else ops.LAUNCHES
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.__enter__()
        ms = event_ms(one, n_steps)
        if sampler:
            sampler.__exit__()
        launches = (ops.LAUNCHES + runner.graph_launches if hasattr(runner, "graph_launches") else ops.LAUNCHES) - launches0
        mean_ctx = PROMPT_LEN + warmup + n_steps / 2
        for rid in ids:
            runner.end_request(rid)
        return ms / n_steps, launches, mean_ctx, (sampler.summary() if sampler else None)

    ms_step, launches, mean_ctx, clocks = decode_point(args.batch, steps, sample_clocks=True)
    value = args.batch / (ms_step * 1e-3)
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_bytes_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            m, _, _, _ = decode_point(b, min(steps, 32))
            points[f"decode_b{b}"] = round(b / (m * 1e-3), 1)

    # ------------------------------------------------- end to end through the API
    def e2e_point(batch: int, n_steps: int, **sampling) -> tuple[float, int]:
        """Decoded tokens a second through Engine.step (host tokens in and out), and the bytes of
        the step's one host->device copy.  Greedy unless sampling options are given.  Prompts are
        admitted one a step, so the first request has decoded `batch` tokens before the last one is
        in: every request may generate enough to stay live through the timed steps, and the tokens
        counted are the ones the requests really gained."""
        params = SamplingParams(**{"temperature": 0.0, **sampling}, max_new_tokens=batch + n_steps + warmup + 8, ignore_eos=True)
        rids = [engine.add_request(rand_tokens(PROMPT_LEN), params) for _ in range(batch)]
        reqs = [engine._live[rid] for rid in rids]
        while any(r.num_computed < len(r.prompt) for r in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        before = sum(len(r.output) for r in reqs)
        t0 = time.perf_counter()
        for _ in range(n_steps):
            engine.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        gained = sum(len(r.output) for r in reqs) - before
        if gained != batch * n_steps or len(engine.scheduler.running) != batch:
            raise RuntimeError(f"e2e at batch {batch}: {gained} tokens in {n_steps} steps, {len(engine.scheduler.running)} requests live")
        h2d_bytes = runner.last_h2d_bytes
        while engine.has_unfinished():
            engine.step()
        return gained / dt, int(h2d_bytes)

    e2e_value, h2d = e2e_point(args.batch, steps)
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch}
    if not args.skip_points:
        e2e["points"] = {f"decode_b{b}": round(e2e_point(b, min(steps, 32))[0], 1) for b in (1, 64)}
        # the same with the reference's default sampling options instead of greedy (src/app/cli/args.zig:364-370)
        e2e["sampled"] = {"value": round(e2e_point(args.batch, min(steps, 32), temperature=0.7, top_k=20, top_p=0.8,
                                                   repetition_penalty=1.1, seed=7)[0], 1),
                          "options": "temperature 0.7, top-k 20, top-p 0.8, repetition penalty 1.1"}

    # -------------------------------- where the time goes (uncaptured, never a timed number)
    if args.profile:
        ids = [f"p{i}" for i in range(args.batch)]
        for rid in ids:
            runner.step([StepEntry(rid, rand_tokens(PROMPT_LEN), [])])
        cur = torch.randint(0, cfg.vocab_size, (args.batch,), generator=gen).tolist()
        with engine.profile(hbm_gbs, bf16_tflops) as prof:
            for _ in range(4):
                runner.step_argmax([StepEntry(rid, [t], [0]) for rid, t in zip(ids, cur)])
            decode_profile = prof.summary()
        for rid in ids:
            runner.end_request(rid)
        with engine.profile(hbm_gbs, bf16_tflops) as prof:
            prefill_once()
            prefill_profile = prof.summary()
        with open(args.profile, "w") as f:
            json.dump({"decode": {"batch": args.batch, "context": PROMPT_LEN, **decode_profile},
                       "prefill": {"tokens": PREFILL_TOKENS, **prefill_profile}}, f, indent=1)

    out = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, bf16)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "zinfer_b200",
        "config": {
            "model": "Qwen3-8B shape, random weights", "global_batch": args.batch, "seq_len": CONTEXT_LEN,
            "prompt_len": PROMPT_LEN, "parallelism": "single GPU", "layers": n_layers, "layers_full_model": full_layers,
            "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
            "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "vocab_size": cfg.vocab_size, "page_size": 16, "kv_dtype": "bf16",
            "l2": "inputs larger than L2 (weights streamed every step)", "peaks": peak_src,
        },
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
    }
    ops.require_kernel_status_ok("bench")   # a kernel whose bounded wait ran out would make every number above void
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
