"""Fills a model's declared tensors from a model folder's safetensors file or shards, by tensor name.

The model declares every tensor it needs (name, shape, optional or not).  The
loader compares that list with the file and raises ONE error naming all missing
tensors, all unexpected ones and all wrong shapes.  Floating tensors are kept in
the run's dtype (bfloat16, or float32 for the 32-bit path); a tensor the file
stores in 32-bit stays 32-bit in a bfloat16 run; integer tables become int32.

The reference resolves each tensor by name once at start
(src/model/runtime/optimized_decoder/layer.zig:81-87) and fails on the first name
it does not find (src/tensor/storage/store.zig:35-45).
"""
from __future__ import annotations

import torch

from ..parts.base import TensorSpec
from .checkpoint import Checkpoint


class WeightsError(ValueError):
    def __init__(self, path: str, missing: list[str], unexpected: list[str], wrong_shape: list[str],
                 wrong_kind: list[str] = ()):
        self.missing, self.unexpected, self.wrong_shape, self.wrong_kind = missing, unexpected, wrong_shape, list(wrong_kind)
        lines = [f"{path} does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong element types ({len(self.wrong_kind)}): " + "; ".join(self.wrong_kind))
        super().__init__("\n".join(lines))


def kept_dtype(stored: torch.dtype, spec: TensorSpec, run_dtype: torch.dtype) -> torch.dtype:
    if spec.integer:
        return torch.int32
    if run_dtype == torch.float32 or stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_against(path: str, available: dict[str, tuple[tuple[int, ...], torch.dtype]],
                  specs: dict[str, TensorSpec]) -> None:
    missing = [n for n, s in specs.items() if n not in available and not s.optional]
    unexpected = [n for n in available if n not in specs]
    wrong, kind = [], []
    for n, s in specs.items():
        if n in available:
            shape, dt = available[n]
            if tuple(shape) != tuple(s.shape):
                wrong.append(f"{n}: file has {list(shape)}, model needs {list(s.shape)}")
            if s.integer == dt.is_floating_point:
                kind.append(f"{n}: file has {dt}, model needs {'an integer' if s.integer else 'a floating'} type")
    if missing or unexpected or wrong or kind:
        raise WeightsError(path, sorted(missing), sorted(unexpected), wrong, kind)


def load_tensors(model_dir: str, specs: dict[str, TensorSpec], run_dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    """One error (:class:`WeightsError`) for everything missing, unexpected or misshapen, over
    all shards together; then every declared tensor is copied to ``device``, shard by shard."""
    with Checkpoint(model_dir) as ck:
        available = ck.available()
        check_against(ck.path, available, specs)
        out = {}
        # shard by shard, so that each mapping is walked once from front to back
        for name in sorted((n for n in specs if n in available), key=lambda n: (ck.where[n], ck.info(n).begin)):
            src = ck.tensor(name)
            dt = kept_dtype(src.dtype, specs[name], run_dtype)
            out[name] = src.to(device=device, dtype=dt, copy=True)
        return {n: out[n] for n in specs if n in out}
