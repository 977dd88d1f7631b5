"""Random weights from a configuration and a seed.

Matrices are normal(0, 0.02) and norm weights 1 + U(-0.1, 0.1).  Each tensor has a
generator of its own, seeded by the seed and the tensor's name, so a tensor's
values do not depend on which other tensors the model has.  ``write_model_dir``
writes a model folder (config.json, model.safetensors) that the loader reads back;
``random_tensors`` fills the tensors in place on a device, for models too large to
pass through a file (the benchmark's).
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from ..parts.base import TensorSpec
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, name))
    if spec.integer:
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "norm":
        t = 1.0 + (torch.rand(spec.shape, generator=gen, device=device, dtype=torch.float32) * 0.2 - 0.1)
    elif spec.init == "zeros":
        t = torch.zeros(spec.shape, device=device, dtype=torch.float32)
    else:
        if len(spec.shape) >= 2 and spec.shape[0] * spec.shape[1] > (1 << 26):
            # large matrices are drawn in row blocks to bound the 32-bit staging buffer
            t = torch.empty(spec.shape, dtype=dtype, device=device)
            rows = max(1, (1 << 26) // spec.shape[1])
            for r0 in range(0, spec.shape[0], rows):
                blk = t[r0:r0 + rows]
                blk.copy_(torch.randn(blk.shape, generator=gen, device=device, dtype=torch.float32) * 0.02)
            return t
        t = torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32) * 0.02
    return t.to(dtype)


def random_tensors(specs: dict[str, TensorSpec], seed: int, dtype: torch.dtype, device="cpu",
                   include_optional: bool = False) -> dict[str, torch.Tensor]:
    return {n: random_tensor(n, s, seed, dtype, device) for n, s in specs.items() if include_optional or not s.optional}


def write_model_dir(path: str, config, seed: int, dtype: torch.dtype = torch.bfloat16, shards: int = 1) -> str:
    """Writes ``config.json`` and ``model.safetensors`` (or, with ``shards`` > 1, that many
    shard files and ``model.safetensors.index.json``) for a typed configuration of a
    registered architecture; returns ``path``.  The tensors do not depend on ``shards``."""
    from ..config.registry import family_for
    from ..engine.model import declared_tensors

    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    fam = family_for(raw)
    specs = declared_tensors(fam.model_spec(config))
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(raw, f, indent=2)
    tensors, meta = random_tensors(specs, seed, dtype), {"format": "pt", "seed": str(seed)}
    if shards > 1:
        from .checkpoint import write_sharded
        write_sharded(path, tensors, shards, metadata=meta)
    else:
        write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata=meta)
    return path
