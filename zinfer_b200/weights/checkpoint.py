"""A model folder's tensors, whether they lie in one file or in shards.

``model.safetensors`` alone, or ``model.safetensors.index.json`` whose
``weight_map`` names the shard file of every tensor
(``{"metadata": {"total_size": n}, "weight_map": {"model.norm.weight": "model-00002-of-00003.safetensors", ...}}``).
Each shard is opened (memory-mapped and validated) once.  The reference reads the
single file only (src/tensor/backends/backend.zig:39); published checkpoints of the
larger models come in shards, so this lifts that limit.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

from .safetensors_io import SafetensorsFile, TensorInfo, write_safetensors

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"


class CheckpointError(ValueError):
    """The folder's files do not form a checkpoint: no weights at all, an index that is not
    valid, shards that the index names but the folder lacks, tensors that the index places in
    a shard which does not hold them, or a tensor held by two shards."""


class Checkpoint:
    """Open shards of one model folder; ``tensor(name)`` gives a CPU view (copy it before ``close``)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files: dict[str, SafetensorsFile] = {}
        self.where: dict[str, str] = {}            # tensor name -> shard file name
        index = os.path.join(model_dir, INDEX_FILE)
        single = os.path.join(model_dir, SINGLE_FILE)
        try:
            if os.path.exists(index):
                self.path = index
                self._open_sharded(index)
            elif os.path.exists(single):
                self.path = single
                self.files[SINGLE_FILE] = SafetensorsFile(single)
                self.where = {n: SINGLE_FILE for n in self.files[SINGLE_FILE].tensors}
            else:
                raise FileNotFoundError(
                    f"{model_dir}: neither {SINGLE_FILE} nor {INDEX_FILE} (a model folder holds config.json and "
                    f"its weights in one of these forms)")
        except Exception:
            self.close()
            raise

    def _open_sharded(self, index: str) -> None:
        try:
            with open(index) as f:
                doc = json.load(f)
        except json.JSONDecodeError as e:
            raise CheckpointError(f"{index}: invalid JSON: {e}") from None
        wm = doc.get("weight_map") if isinstance(doc, dict) else None
        if not isinstance(wm, dict) or not wm or any(not isinstance(k, str) or not isinstance(v, str) for k, v in wm.items()):
            raise CheckpointError(f"{index}: `weight_map` must map tensor names to shard file names")
        shards = sorted(set(wm.values()))
        absent = [s for s in shards if os.path.basename(s) != s or not os.path.exists(os.path.join(self.model_dir, s))]
        if absent:
            raise CheckpointError(f"{index}: shards named by the index but not in the folder: {', '.join(absent)}")
        for s in shards:
            self.files[s] = SafetensorsFile(os.path.join(self.model_dir, s))
        misplaced = sorted(n for n, s in wm.items() if n not in self.files[s].tensors)
        if misplaced:
            raise CheckpointError(f"{index}: tensors that their shard does not hold: " +
                                  ", ".join(f"{n} ({wm[n]})" for n in misplaced))
        twice = []
        for s, f in self.files.items():
            for n in f.tensors:
                if n in self.where:
                    twice.append(f"{n} ({self.where[n]}, {s})")
                self.where[n] = s
        if twice:
            raise CheckpointError(f"{index}: tensors held by two shards: " + ", ".join(sorted(twice)))

    # ------------------------------------------------------------------ reading
    def info(self, name: str) -> TensorInfo:
        return self.files[self.where[name]].tensors[name]

    def available(self) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        return {n: (self.info(n).shape, self.info(n).torch_dtype) for n in self.where}

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self.where:
            raise KeyError(f"{self.path}: no tensor named {name!r}")
        return self.files[self.where[name]].tensor(name)

    def close(self) -> None:
        for f in self.files.values():
            f.close()
        self.files = {}

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_sharded(model_dir: str, tensors: dict[str, torch.Tensor], shards: int,
                  metadata: Optional[dict[str, str]] = None) -> list[str]:
    """Writes ``tensors`` as ``shards`` files of about equal size (in the order given, never
    splitting a tensor) and the index that names them; returns the shard file names."""
    if shards < 1:
        raise ValueError("shards must be >= 1")
    names = list(tensors)
    sizes = [tensors[n].numel() * tensors[n].element_size() for n in names]
    total, shards = sum(sizes), min(shards, max(1, len(names)))
    groups: list[list[str]] = [[] for _ in range(shards)]
    acc, gi = 0, 0
    for n, sz in zip(names, sizes):
        left_names, left_groups = len(names) - sum(len(g) for g in groups), shards - gi
        if groups[gi] and gi < shards - 1 and (acc >= total * (gi + 1) / shards or left_names <= left_groups - 1):
            gi += 1
        groups[gi].append(n)
        acc += sz
    groups = [g for g in groups if g]
    files = [f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors" for i in range(len(groups))]
    weight_map = {}
    for fname, g in zip(files, groups):
        write_safetensors(os.path.join(model_dir, fname), {n: tensors[n] for n in g}, metadata=metadata)
        weight_map.update({n: fname for n in g})
    with open(os.path.join(model_dir, INDEX_FILE), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    return files
