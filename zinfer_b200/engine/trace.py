"""Trace replay: feeds given token ids through the model step by step and writes
the logits.  It samples nothing and has no forward pass, cache or loader of its
own: it drives :class:`ModelRunner`, the step function generation uses.

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits
at the wanted places, in the order of the entries and of ``want``, as
little-endian 32-bit floats [wanted, vocab].  After every step a line
``done <step>`` is printed and flushed.

The reference's nearest tool feeds ids one by one and prints greedy ids
(src/app/cli/inspect.zig:246-312).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--poison-freed-pages", action="store_true",
                    help="debugging: overwrite every page with huge values when it is given back")
    args = ap.parse_args(argv)

    from .. import ops
    from .batch import StepEntry
    from .runner import ModelRunner

    if args.page_size <= 0 or 64 % args.page_size:
        print("trace_run: --page-size must divide 64", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    runner = ModelRunner.from_model_dir(args.model, dtype=dtype, device=args.device, page_size=args.page_size,
                                        max_tokens=max(args.max_tokens, args.page_size), max_requests=64,
                                        poison_freed_pages=args.poison_freed_pages)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", [])]
        logits = runner.step(entries)
        if logits is not None:
            arr = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
            arr.tofile(os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            if runner.has_request(rid):
                runner.end_request(rid)
        ops.require_kernel_status_ok(f"step {step}")   # a kernel whose bounded wait ran out fails the replay
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    reused = sum(g.pool.reused for g in runner.manager.groups)
    print(f"trace_run: {runner.steps_run} steps, {reused} page allocations returned a page used before", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
