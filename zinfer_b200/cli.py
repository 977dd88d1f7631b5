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
  zinfer generate [model_dir] <ids_csv> [max_new_tokens] [flags...]
  zinfer bench [model_dir] <ids_csv> [max_new_tokens] [flags...]
  zinfer bench-batch [model_dir] <ids_csv> <batch_size> [max_new_tokens] [flags...]
  zinfer bench-continuous [model_dir] <ids_csv> <batch_size> <total_requests> [max_new_tokens] [flags...]
  zinfer random-model <out_dir> <config_json> [seed]

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
  --ignore-eos
  --dtype <bfloat16|float32>
  --page-size <usize>
  --kv-cache-tokens <usize>
  --max-batched-tokens <usize>
  --chunk-size <usize>
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
}


def parse_flags(args: list[str]) -> tuple[dict, dict]:
    """(sampling options, engine options); errors carry the reference's names
    (MissingFlagValue, UnknownFlag, args.zig:395-501)."""
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
        table = _FLAGS if a in _FLAGS else _ENGINE_FLAGS if a in _ENGINE_FLAGS else None
        if table is None:
            raise CliError(f"UnknownFlag: {a}")
        if i + 1 >= len(args):
            raise CliError(f"MissingFlagValue: {a}")
        key, conv = table[a]
        try:
            (sampling if table is _FLAGS else engine)[key] = conv(args[i + 1])
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
    from .weights import SafetensorsFile

    path = os.path.join(model_dir, "model.safetensors")
    with SafetensorsFile(path) as f:
        print("Zinfer weights inspection", file=out)
        print(f"weights_path: {path}", file=out)
        print(f"file_size: {os.path.getsize(path)}", file=out)
        print(f"header_len: {f.data_start - 8}", file=out)
        print(f"data_start: {f.data_start}", file=out)
        print(f"tensor_count: {len(f.tensors)}", file=out)
        for k, v in f.metadata.items():
            print(f"metadata.{k}: {v}", file=out)
        for name, t in f.tensors.items():
            print(f"tensor {name}: dtype={t.dtype} shape={list(t.shape)} bytes={t.end - t.begin}", file=out)


def inspect_tensor(model_dir: str, name: str, count: int, out) -> None:
    from .weights import SafetensorsFile

    with SafetensorsFile(os.path.join(model_dir, "model.safetensors")) as f:
        if name not in f.tensors:
            raise CliError(f"TensorNotFound: {name}")
        info = f.tensors[name]
        vals = f.tensor(name).reshape(-1)[:count].float().tolist()
        print(f"tensor: {name}", file=out)
        print(f"dtype: {info.dtype}", file=out)
        print(f"shape: {list(info.shape)}", file=out)
        for i, v in enumerate(vals):
            print(f"value[{i}]: {v:.8f}", file=out)


def _engine(model_dir: str, engine_opts: dict, **defaults):
    from .engine.api import Engine

    opts = {**defaults, **engine_opts}
    return Engine(model_dir, **opts)


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


def generate(model_dir: str, ids_csv: str, max_new: int, sampling: dict, engine_opts: dict, out) -> None:
    from .sampling import SamplingParams

    ids = parse_token_ids(ids_csv)
    if not ids:
        raise CliError("EmptyPrompt")
    eng = _engine(model_dir, engine_opts, max_requests=1, kv_cache_tokens=len(ids) + max_new + 64)
    res = eng.generate([ids], SamplingParams(max_new_tokens=max_new, **sampling))[0]
    print("tokens: [" + ", ".join(str(t) for t in res.token_ids) + "]", file=out)
    print(f"finish_reason: {res.finish_reason}", file=out)


def bench(model_dir: str, ids_csv: str, batch: int, total: int, max_new: int, sampling: dict, engine_opts: dict,
          out) -> None:
    """Prefill and decode rates in the reference's key: value style
    (src/app/cli/tools/bench/runtime.zig:80-98,198-223,284-309)."""
    import torch
    from .sampling import SamplingParams

    ids = parse_token_ids(ids_csv)
    if not ids:
        raise CliError("EmptyPrompt")
    eng = _engine(model_dir, engine_opts, max_requests=batch, kv_cache_tokens=batch * (len(ids) + max_new + 64))
    params = SamplingParams(max_new_tokens=max_new, **{"temperature": 0.0, "ignore_eos": True, **sampling})
    eng.generate([ids], params, max_new_tokens=2)   # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    results = eng.generate([ids] * total, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.scheduler.stats
    decoded = sum(len(r.token_ids) for r in results)
    print("Zinfer benchmark", file=out)
    print(f"model_dir: {model_dir}", file=out)
    print(f"batch_size: {batch}", file=out)
    print(f"total_requests: {total}", file=out)
    print(f"prompt_tokens: {len(ids)}", file=out)
    print(f"decoded_tokens: {decoded}", file=out)
    print(f"total_ms: {dt * 1e3:.3f}", file=out)
    print(f"total_tok_s: {(decoded + total * len(ids)) / dt:.2f}", file=out)
    print(f"decode_tok_s: {decoded / dt:.2f}", file=out)
    print(f"preemptions: {st.preemptions}", file=out)
    print(f"weights_bytes: {eng.runner.model.weight_bytes()}", file=out)
    print(f"kv_cache_bytes: {eng.runner.storage.bytes()}", file=out)


def random_model(out_dir: str, config_json: str, seed: int, out) -> None:
    from .config.registry import family_for
    from .weights import write_model_dir

    with open(config_json) as f:
        raw = json.load(f)
    cfg = family_for(raw).config_class.from_dict(raw)
    write_model_dir(out_dir, cfg, seed)
    print(f"wrote {out_dir} (seed {seed})", file=out)


# --------------------------------------------------------------------------- main
def run(argv: list[str], out=sys.stdout) -> int:
    if not argv or argv[0] in ("-h", "--help", "help"):
        out.write(USAGE)
        return 0
    cmd, rest = argv[0], argv[1:]
    try:
        if cmd == "random-model":
            pos, _ = _positionals(rest)
            if len(pos) < 2:
                raise CliError("InvalidCommand")
            random_model(pos[0], pos[1], _int(pos[2], "seed") if len(pos) > 2 else 0, out)
            return 0
        model_dir, rest = split_model_dir(rest)
        pos, flags = _positionals(rest)
        sampling, engine_opts = parse_flags(flags)
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
            probe_model(model_dir, _int(pos[0], "token_id"), _int(pos[1], "top_k"), engine_opts, out)
        elif cmd == "generate-token-ids":
            if len(pos) < 2:
                raise CliError("InvalidCommand")
            generate_token_ids(model_dir, pos[0], _int(pos[1], "steps"), engine_opts, out)
        elif cmd == "generate":
            if not pos:
                raise CliError("InvalidCommand")
            generate(model_dir, pos[0], _int(pos[1], "max_new_tokens") if len(pos) > 1 else 64, sampling, engine_opts, out)
        elif cmd == "bench":
            if not pos:
                raise CliError("InvalidCommand")
            bench(model_dir, pos[0], 1, 1, _int(pos[1], "max_new_tokens") if len(pos) > 1 else 16, sampling, engine_opts, out)
        elif cmd == "bench-batch":
            if len(pos) < 2:
                raise CliError("InvalidCommand")
            b = _int(pos[1], "batch_size")
            bench(model_dir, pos[0], b, b, _int(pos[2], "max_new_tokens") if len(pos) > 2 else 16, sampling, engine_opts, out)
        elif cmd == "bench-continuous":
            if len(pos) < 3:
                raise CliError("InvalidCommand")
            bench(model_dir, pos[0], _int(pos[1], "batch_size"), _int(pos[2], "total_requests"),
                  _int(pos[3], "max_new_tokens") if len(pos) > 3 else 16, sampling, engine_opts, out)
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
