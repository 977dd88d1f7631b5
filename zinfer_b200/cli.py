"""The command line, in the reference's manner: positional sub-commands with an
optional model folder first, then ``--flag value`` options with the reference's
names and meanings (src/app/cli/usage.zig:6-65, src/app/cli/args.zig:395-501).
The engine works on token ids, so where the reference takes text this takes ids
as ``1,2,3`` (its own ``generate-token-ids`` form, src/app/cli/token_ids.zig:3-18).
"""
from __future__ import annotations

import json
import os
import sys
import time

DEFAULT_MODEL_DIR = "models/Qwen3-0.6B"   # src/app/cli/args.zig:7

USAGE = """Usage:
  zinfer inspect-config [model_dir]
  zinfer inspect-weights [model_dir]
  zinfer inspect-tensor [model_dir] <tensor_name> [count]
  zinfer probe-model [model_dir] <token_id> <top_k>
  zinfer generate-token-ids [model_dir] <seed_ids_csv> <steps>
  zinfer generate [model_dir] <ids_csv[;ids_csv...]> [max_new_tokens] [flags...]
  zinfer bench [model_dir] <ids_csv> [max_new_tokens] [flags...]
  zinfer bench-batch [model_dir] <ids_csv> <batch_size> [max_new_tokens] [flags...]
  zinfer bench-continuous [model_dir] <ids_csv> <batch_size> <total_requests> [max_new_tokens] [flags...]
  zinfer random-model <out_dir> <config_json> [seed] [--shards <usize>]

  Instead of [model_dir], `--random-weights <seed> --config <config_json>` draws the
  weights on the GPU (no folder is read or written).  Several prompts, separated by
  `;`, run as one batch.

Defaults:
  model_dir = models/Qwen3-0.6B
  generate max_new_tokens = 64
  bench max_new_tokens = 16

Flags:
  --seed <u64>
  --temperature <f32>
  --top-p <f32>
  --top-k <usize>
  --min-p <f32>
  --presence-penalty <f32>
  --frequency-penalty <f32>
  --repetition-penalty <f32>
  --max-new-tokens <usize>     (same as the positional)
  --ignore-eos
  --stop <ids_csv>             (repeatable: generation ends when the generated ids end with these; they are not
                                part of the response)
  --stream                     (generate: print ids as they are generated, `stream[i]: ...`, holding back a tail
                                that may still become a stop sequence)
  --dtype <bfloat16|float32>
  --device <cuda:N>
  --random-weights <seed>      (with --config)
  --config <config_json>
  --page-size <usize>
  --num-pages <usize>          (pages per cache group; else:)
  --kv-cache-tokens <usize>    (else:)
  --kv-cache-bytes <usize>     (else: --gpu-memory-fraction of what is free, default 0.9)
  --gpu-memory-fraction <f32>
  --max-model-len <usize>
  --max-requests <usize>
  --max-batched-tokens <usize>
  --chunk-size <usize>
  --profile <path>             (generate, bench*: per-kernel-class device times as JSON;
                                with --hbm-gbs <f32> --bf16-tflops <f32> also fractions of those peaks)
"""


class CliError(Exception):
    pass


def parse_token_ids(csv: str) -> list[int]:
    """"1,2,3" -> [1, 2, 3]; blanks around numbers are allowed (token_ids.zig:3-18)."""
    out = []
    for part in csv.split(","):
        part = part.strip()
        if not part:
            continue
        try:
            v = int(part)
        except ValueError:
            raise CliError(f"InvalidTokenId: {part!r}") from None
        if v < 0:
            raise CliError(f"InvalidTokenId: {part!r}")
        out.append(v)
    return out


_FLAGS = {
    "--seed": ("seed", int), "--temperature": ("temperature", float), "--top-p": ("top_p", float),
    "--top-k": ("top_k", int), "--min-p": ("min_p", float), "--presence-penalty": ("presence_penalty", float),
    "--frequency-penalty": ("frequency_penalty", float), "--repetition-penalty": ("repetition_penalty", float),
}
_ENGINE_FLAGS = {
    "--dtype": ("dtype", str), "--page-size": ("page_size", int), "--kv-cache-tokens": ("kv_cache_tokens", int),
    "--max-batched-tokens": ("max_batched_tokens", int), "--chunk-size": ("chunk_size", int),
    "--num-pages": ("num_pages", int), "--kv-cache-bytes": ("kv_cache_bytes", int),
    "--gpu-memory-fraction": ("gpu_memory_fraction", float), "--max-model-len": ("max_model_len", int),
    "--max-requests": ("max_requests", int), "--device": ("device", str),
}
# options of the command itself: where the model comes from, how much to generate, what to record
_RUN_FLAGS = {
    "--random-weights": ("random_weights", int), "--config": ("config", str), "--max-new-tokens": ("max_new_tokens", int),
    "--profile": ("profile", str), "--shards": ("shards", int), "--hbm-gbs": ("hbm_gbs", float),
    "--bf16-tflops": ("bf16_tflops", float),
}


def parse_flags(args: list[str], run_opts: dict | None = None) -> tuple[dict, dict]:
    """(sampling options, engine options); options of the command itself go to ``run_opts``
    when given.  Errors carry the reference's names (MissingFlagValue, UnknownFlag,
    args.zig:395-501)."""
    sampling, engine = {}, {}
    i = 0
    while i < len(args):
        a = args[i]
        if not a.startswith("--"):
            raise CliError(f"InvalidCommand: expected a flag, got {a!r}")
        if a == "--ignore-eos":
            sampling["ignore_eos"] = True
            i += 1
            continue
        if a == "--stream" and run_opts is not None:
            run_opts["stream"] = True
            i += 1
            continue
        if a == "--stop":                       # repeatable, like the reference's (args.zig:462-466); ids instead of text
            if i + 1 >= len(args):
                raise CliError(f"MissingFlagValue: {a}")
            sampling.setdefault("stop_sequences", []).append(parse_token_ids(args[i + 1]))
            i += 2
            continue
        table = (_FLAGS if a in _FLAGS else _ENGINE_FLAGS if a in _ENGINE_FLAGS
                 else _RUN_FLAGS if a in _RUN_FLAGS and run_opts is not None else None)
        if table is None:
            raise CliError(f"UnknownFlag: {a}")
        if i + 1 >= len(args):
            raise CliError(f"MissingFlagValue: {a}")
        key, conv = table[a]
        try:
            (sampling if table is _FLAGS else engine if table is _ENGINE_FLAGS else run_opts)[key] = conv(args[i + 1])
        except ValueError:
            raise CliError(f"InvalidFlagValue: {a} {args[i + 1]!r}") from None
        i += 2
    return sampling, engine


def split_model_dir(args: list[str]) -> tuple[str, list[str]]:
    """The first positional is the model folder if it holds a config.json."""
    if args and not args[0].startswith("--") and os.path.isfile(os.path.join(args[0], "config.json")):
        return args[0], args[1:]
    return DEFAULT_MODEL_DIR, args


def _positionals(args: list[str]) -> tuple[list[str], list[str]]:
    n = next((i for i, a in enumerate(args) if a.startswith("--")), len(args))
    return args[:n], args[n:]


def _int(value: str, what: str) -> int:
    try:
        return int(value)
    except ValueError:
        raise CliError(f"InvalidCommand: {what} must be an integer, got {value!r}") from None


# ------------------------------------------------------------------- sub-commands
def inspect_config(model_dir: str, out) -> None:
    from .config.registry import load_config

    fam, cfg = load_config(model_dir)
    print("Zinfer model inspection", file=out)
    print(f"model_dir: {model_dir}", file=out)
    print(f"model_type: {cfg.model_type}", file=out)
    print(f"architecture: {fam.name}", file=out)
    for k in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
              "head_dim", "vocab_size", "max_position_embeddings"):
        print(f"{k}: {getattr(cfg, k)}", file=out)
    print(f"rope_theta: {int(cfg.rope_theta)}", file=out)
    print(f"rms_norm_eps: {cfg.rms_norm_eps:e}", file=out)
    print(f"torch_dtype: {cfg.torch_dtype}", file=out)
    print(f"tie_word_embeddings: {str(cfg.tie_word_embeddings).lower()}", file=out)


def inspect_weights(model_dir: str, out) -> None:
    from .weights import Checkpoint

    with Checkpoint(model_dir) as ck:
        print("Zinfer weights inspection", file=out)
        for fname, f in ck.files.items():
            print(f"weights_path: {f.path}", file=out)
            print(f"file_size: {os.path.getsize(f.path)}", file=out)
            print(f"header_len: {f.data_start - 8}", file=out)
            print(f"data_start: {f.data_start}", file=out)
            for k, v in f.metadata.items():
                print(f"metadata.{k}: {v}", file=out)
        print(f"shard_count: {len(ck.files)}", file=out)
        print(f"tensor_count: {len(ck.where)}", file=out)
        for name in ck.where:
            t = ck.info(name)
            print(f"tensor {name}: dtype={t.dtype} shape={list(t.shape)} bytes={t.end - t.begin}", file=out)


def inspect_tensor(model_dir: str, name: str, count: int, out) -> None:
    from .weights import Checkpoint

    with Checkpoint(model_dir) as ck:
        if name not in ck.where:
            raise CliError(f"TensorNotFound: {name}")
        info = ck.info(name)
        vals = ck.tensor(name).reshape(-1)[:count].float().tolist()
        print(f"tensor: {name}", file=out)
        print(f"dtype: {info.dtype}", file=out)
        print(f"shape: {list(info.shape)}", file=out)
        for i, v in enumerate(vals):
            print(f"value[{i}]: {v:.8f}", file=out)


class ModelSource:
    """Where the weights come from: a model folder, or a configuration file and a seed
    (``--random-weights <seed> --config <config_json>``: drawn on the GPU, nothing read or written)."""

    def __init__(self, model_dir: str | None, run_opts: dict):
        self.seed = run_opts.get("random_weights")
        self.config_path = run_opts.get("config")
        if (self.seed is None) != (self.config_path is None):
            raise CliError("InvalidCommand: --random-weights <seed> and --config <config_json> go together")
        self.model_dir = None if self.seed is not None else model_dir

    @property
    def label(self) -> str:
        return self.model_dir if self.model_dir is not None else f"{self.config_path} (random weights, seed {self.seed})"

    def engine(self, engine_opts: dict, **defaults):
        from .engine.api import Engine

        opts = {**defaults, **engine_opts}
        if any(k in engine_opts for k in ("num_pages", "kv_cache_bytes", "kv_cache_tokens", "gpu_memory_fraction")):
            for k in ("num_pages", "kv_cache_bytes", "kv_cache_tokens"):     # the user's choice of pool beats the command's default
                if k not in engine_opts:
                    opts.pop(k, None)
        if self.model_dir is not None:
            return Engine(self.model_dir, **opts)
        from .config.registry import family_for

        with open(self.config_path) as f:
            raw = json.load(f)
        return Engine(config=family_for(raw).config_class.from_dict(raw), random_weights_seed=self.seed, **opts)


def _engine(model, engine_opts: dict, **defaults):
    if isinstance(model, str):
        model = ModelSource(model, {})
    return model.engine(engine_opts, **defaults)


def _profiled(run_opts: dict, eng, fn):
    """Runs ``fn()``; with ``--profile <path>`` under the profiler, whose summary goes to that file."""
    path = run_opts.get("profile")
    if not path:
        return fn()
    with eng.profile(run_opts.get("hbm_gbs"), run_opts.get("bf16_tflops")) as prof:
        res = fn()
    prof.dump(path)
    return res


def _pool_lines(eng, out) -> None:
    from .cache import bytes_per_token

    kv_needs, _ = eng.runner.model.cache_needs()
    elt = eng.runner.model.dtype.itemsize
    print(f"weights_bytes: {eng.runner.model.weight_bytes()}", file=out)
    print(f"kv_cache_bytes: {eng.runner.storage.bytes()}", file=out)
    print(f"kv_bytes_per_token: {bytes_per_token(kv_needs, elt)}", file=out)
    print(f"num_pages: {eng.runner.manager.groups[0].pool.num_pages if eng.runner.manager.groups else 0}", file=out)
    print(f"page_size: {eng.runner.manager.page_size}", file=out)


def probe_model(model_dir: str, token_id: int, top_k: int, engine_opts: dict, out) -> None:
    """Top-k logits after one token (src/app/cli/inspect.zig:206-244)."""
    import torch
    from .engine import StepEntry

    eng = _engine(model_dir, engine_opts, max_requests=1, kv_cache_tokens=64)
    logits = eng.runner.step([StepEntry("probe", [token_id], [0])])[0]
    vals, idx = torch.topk(logits, min(top_k, logits.numel()))
    print("Zinfer model probe", file=out)
    print(f"token_id: {token_id}", file=out)
    for v, i in zip(vals.tolist(), idx.tolist()):
        print(f"top_logit token={i} value={v:.6f}", file=out)


def generate_token_ids(model_dir: str, ids_csv: str, steps: int, engine_opts: dict, out) -> None:
    """Greedy continuation of given ids; prints ids (src/app/cli/inspect.zig:246-312)."""
    from .sampling import SamplingParams

    seed_ids = parse_token_ids(ids_csv)
    if not seed_ids:
        raise CliError("EmptySeed")
    eng = _engine(model_dir, engine_opts, max_requests=1, kv_cache_tokens=len(seed_ids) + steps + 64)
    res = eng.generate([seed_ids], SamplingParams(temperature=0.0, max_new_tokens=steps, ignore_eos=True))[0]
    print("Zinfer generated token ids", file=out)
    print(f"seed: {ids_csv}", file=out)
    print(f"steps: {steps}", file=out)
    print("tokens: [" + ", ".join(str(t) for t in seed_ids + res.token_ids) + "]", file=out)


def generate(model, ids_csv: str, max_new: int, sampling: dict, engine_opts: dict, out, run_opts: dict | None = None) -> None:
    """One prompt, or several separated by ``;`` that run as one batch (ids in, ids out)."""
    from .sampling import SamplingParams

    prompts = [parse_token_ids(part) for part in ids_csv.split(";") if part.strip()]
    if not prompts or any(not p for p in prompts):
        raise CliError("EmptyPrompt")
    page = engine_opts.get("page_size", 16)
    eng = _engine(model, engine_opts, max_requests=max(1, len(prompts)),
                  kv_cache_tokens=sum(-(-(len(p) + max_new) // page) * page + page for p in prompts))
    params = SamplingParams(max_new_tokens=max_new, **sampling)

    def streamed():
        done = {}
        for i, new_ids, res in eng.generate_stream(prompts, params):
            if new_ids:
                print(f"stream[{i}]: " + " ".join(str(t) for t in new_ids), file=out, flush=True)
            if res is not None:
                done[i] = res
        return [done[i] for i in range(len(prompts))]

    results = _profiled(run_opts or {}, eng, streamed if (run_opts or {}).get("stream") else lambda: eng.generate(prompts, params))
    for i, res in enumerate(results):
        tag = "" if len(results) == 1 else f"[{i}]"
        print(f"tokens{tag}: [" + ", ".join(str(t) for t in res.token_ids) + "]", file=out)
        print(f"finish_reason{tag}: {res.finish_reason}", file=out)


def bench(model, ids_csv: str, batch: int, total: int, max_new: int, sampling: dict, engine_opts: dict,
          out, run_opts: dict | None = None) -> None:
    """Prefill and decode rates in the reference's key: value style
    (src/app/cli/tools/bench/runtime.zig:80-98,198-223,284-309)."""
    import torch
    from .sampling import SamplingParams

    ids = parse_token_ids(ids_csv)
    if not ids:
        raise CliError("EmptyPrompt")
    model = model if isinstance(model, ModelSource) else ModelSource(model, {})
    eng = _engine(model, engine_opts, max_requests=batch, kv_cache_tokens=batch * (len(ids) + max_new + 64))
    params = SamplingParams(max_new_tokens=max_new, **{"temperature": 0.0, "ignore_eos": True, **sampling})
    eng.generate([ids], params, max_new_tokens=2)   # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    results = _profiled(run_opts or {}, eng, lambda: eng.generate([ids] * total, params))
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.scheduler.stats
    decoded = sum(len(r.token_ids) for r in results)
    print("Zinfer benchmark", file=out)
    print(f"model_dir: {model.label}", file=out)
    print(f"batch_size: {batch}", file=out)
    print(f"total_requests: {total}", file=out)
    print(f"prompt_tokens: {len(ids)}", file=out)
    print(f"decoded_tokens: {decoded}", file=out)
    print(f"total_ms: {dt * 1e3:.3f}", file=out)
    print(f"total_tok_s: {(decoded + total * len(ids)) / dt:.2f}", file=out)
    print(f"decode_tok_s: {decoded / dt:.2f}", file=out)
    print(f"preemptions: {st.preemptions}", file=out)
    _pool_lines(eng, out)


def random_model(out_dir: str, config_json: str, seed: int, out, shards: int = 1) -> None:
    from .config.registry import family_for
    from .weights import write_model_dir

    with open(config_json) as f:
        raw = json.load(f)
    cfg = family_for(raw).config_class.from_dict(raw)
    write_model_dir(out_dir, cfg, seed, shards=shards)
    print(f"wrote {out_dir} (seed {seed}" + (f", {shards} shards)" if shards > 1 else ")"), file=out)


# --------------------------------------------------------------------------- main
def run(argv: list[str], out=sys.stdout) -> int:
    if not argv or argv[0] in ("-h", "--help", "help"):
        out.write(USAGE)
        return 0
    cmd, rest = argv[0], argv[1:]
    try:
        if cmd == "random-model":
            pos, flags = _positionals(rest)
            run_opts: dict = {}
            parse_flags(flags, run_opts)
            if len(pos) < 2:
                raise CliError("InvalidCommand")
            random_model(pos[0], pos[1], _int(pos[2], "seed") if len(pos) > 2 else 0, out, shards=run_opts.get("shards", 1))
            return 0
        model_dir, rest = split_model_dir(rest)
        pos, flags = _positionals(rest)
        run_opts = {}
        sampling, engine_opts = parse_flags(flags, run_opts)
        model = ModelSource(model_dir, run_opts)

        def max_new(index: int, default: int) -> int:
            """The positional at ``index`` if present, else --max-new-tokens, else the command's default."""
            if len(pos) > index:
                return _int(pos[index], "max_new_tokens")
            return run_opts.get("max_new_tokens", default)

        if cmd in ("inspect-config", "inspect-weights", "inspect-tensor") and model.model_dir is None:
            raise CliError("InvalidCommand: inspection needs a model folder")
        if cmd == "inspect-config":
            inspect_config(model_dir, out)
        elif cmd == "inspect-weights":
            inspect_weights(model_dir, out)
        elif cmd == "inspect-tensor":
            if not pos:
                raise CliError("InvalidCommand")
            inspect_tensor(model_dir, pos[0], _int(pos[1], "count") if len(pos) > 1 else 8, out)
        elif cmd == "probe-model":
            if len(pos) < 2:
                raise CliError("InvalidCommand")
            probe_model(model, _int(pos[0], "token_id"), _int(pos[1], "top_k"), engine_opts, out)
        elif cmd == "generate-token-ids":
            if len(pos) < 2:
                raise CliError("InvalidCommand")
            generate_token_ids(model, pos[0], _int(pos[1], "steps"), engine_opts, out)
        elif cmd == "generate":
            if not pos:
                raise CliError("InvalidCommand")
            generate(model, pos[0], max_new(1, 64), sampling, engine_opts, out, run_opts)
        elif cmd == "bench":
            if not pos:
                raise CliError("InvalidCommand")
            bench(model, pos[0], 1, 1, max_new(1, 16), sampling, engine_opts, out, run_opts)
        elif cmd == "bench-batch":
            if len(pos) < 2:
                raise CliError("InvalidCommand")
            b = _int(pos[1], "batch_size")
            bench(model, pos[0], b, b, max_new(2, 16), sampling, engine_opts, out, run_opts)
        elif cmd == "bench-continuous":
            if len(pos) < 3:
                raise CliError("InvalidCommand")
            bench(model, pos[0], _int(pos[1], "batch_size"), _int(pos[2], "total_requests"), max_new(3, 16), sampling,
                  engine_opts, out, run_opts)
        else:
            print(f"error: unknown command {cmd!r}", file=sys.stderr)
            out.write(USAGE)
            return 2
    except CliError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    except (OSError, ValueError, RuntimeError, KeyError) as e:
        print(f"error: {type(e).__name__}: {e}", file=sys.stderr)
        return 1
    return 0


def main() -> int:
    return run(sys.argv[1:])


if __name__ == "__main__":
    sys.exit(main())
