"""A decoder assembled from a :class:`ModelSpec`: embedding, the scheduled runs of
its layers, final norm, output head.  The model knows nothing of Qwen3; the family
function decided the parts and their parameters
(the reference's stack: src/model/layers/decoder_only_stack.zig:48-93).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..cache.storage import CacheStorage
from ..config.spec import ModelSpec
from ..parts.base import BuildContext, KVCacheNeed, StateNeed, TensorSpec, make_part, prefixed, take


@dataclass(frozen=True)
class Run:
    """One scheduled execution of a layer with the cache it uses."""

    layer: int
    cache: str
    writes: bool


def _plan_runs(spec: ModelSpec) -> list[Run]:
    runs, seen = [], set()
    for i, e in enumerate(spec.schedule):
        name = e.cache if e.cache is not None else f"run{i}"
        runs.append(Run(e.layer, name, writes=name not in seen))
        seen.add(name)
    return runs


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, max_positions: Optional[int] = None):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.max_positions = min(spec.max_positions, max_positions) if max_positions else spec.max_positions
        self.ctx = BuildContext(device=self.device, dtype=dtype, max_positions=self.max_positions)
        self.embedding = make_part(spec.embedding, self.ctx)
        self.blocks = [make_part(layer.block, self.ctx) for layer in spec.layers]
        self.final_norm = make_part(spec.final_norm, self.ctx)
        self.head = make_part(spec.head, self.ctx)
        self.runs = _plan_runs(spec)
        self._views: list = []

    # ----------------------------------------------------------------- weights
    def _final_norm_prefix(self) -> str:
        return self.spec.final_norm.params.get("name", "norm") + "."

    def tensor_specs(self) -> dict[str, TensorSpec]:
        out = dict(self.embedding.tensor_specs())
        for layer, block in zip(self.spec.layers, self.blocks):
            out.update(prefixed(layer.prefix, block.tensor_specs()))
        out.update(prefixed(self._final_norm_prefix(), self.final_norm.tensor_specs()))
        out.update(self.head.tensor_specs())
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.embedding.bind(tensors)
        for layer, block in zip(self.spec.layers, self.blocks):
            block.bind(take(tensors, layer.prefix))
        self.final_norm.bind(take(tensors, self._final_norm_prefix()))
        self.head.bind(tensors)
        if getattr(self.head, "tied_to", None) is not None:
            self.head.tie(self.embedding.weight)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for part in [self.embedding, self.final_norm, self.head, *self.blocks]:
            stack = [part]
            while stack:
                p = stack.pop()
                for v in vars(p).values():
                    if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                        seen.add(v.data_ptr())
                        total += v.numel() * v.element_size()
                    elif hasattr(v, "tensor_specs"):
                        stack.append(v)
        return total

    # ------------------------------------------------------------------- caches
    def cache_needs(self) -> tuple[dict[str, KVCacheNeed], dict[str, StateNeed]]:
        kv, state = {}, {}
        for run in self.runs:
            need = self.blocks[run.layer].mixer.cache_need()
            prev = kv.get(run.cache, state.get(run.cache))
            if prev is not None and prev != need:
                raise ValueError(f"cache {run.cache!r} is shared by layers with different needs: {prev} and {need}")
            if isinstance(need, KVCacheNeed):
                kv[run.cache] = need
            elif isinstance(need, StateNeed):
                state[run.cache] = need
            elif need is not None:
                raise TypeError(f"layer {run.layer}: unknown cache need {need!r}")
        return kv, state

    def attach(self, storage: CacheStorage) -> None:
        """Binds every run to its view of the cache storage."""
        kv, state = self.cache_needs()
        self._views = []
        for run in self.runs:
            if run.cache in kv:
                self._views.append(storage.kv_view(run.cache, run.writes))
            elif run.cache in state:
                self._views.append(storage.state_view(run.cache, run.writes))
            else:
                self._views.append(None)

    # ------------------------------------------------------------------ forward
    def forward(self, step, argmax: bool = False):
        """Runs the step's tokens through every scheduled layer (filling the caches)
        and returns 32-bit logits [wanted rows, vocab], or None if none are wanted.
        With ``argmax`` it returns the pair (logits, first maximum of every row as int32)."""
        h = self.embedding.forward(step.token_ids)
        pending = None
        for run, view in zip(self.runs, self._views):
            pending = self.blocks[run.layer].forward(h, pending, step, view)
        if step.logit_rows is None or step.logit_rows.numel() == 0:
            return (None, None) if argmax else None
        x = self.final_norm.forward(h, pending, rows=step.logit_rows)
        if not argmax:
            return self.head.forward(x)
        if hasattr(self.head, "forward_argmax"):     # a head may find the maxima while it makes the logits
            return self.head.forward_argmax(x)
        logits = self.head.forward(x)
        return logits, ops.argmax(logits)


def declared_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """The tensors a model of this spec needs; builds no device memory."""
    return DecoderModel(spec, torch.float32, "cpu").tensor_specs()
