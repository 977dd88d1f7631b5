"""Interfaces of the parts a decoder is put together from, and their registry.

A part is built from the parameters of its :class:`PartSpec` alone; it learns its
sizes and constants there and never which model it is in.  It declares the tensors
it needs by names relative to itself; the model prefixes them and the loader fills
them by name.

Kinds of part and what each must provide:

``Norm``            ``forward(h, delta, rows=None)``: adds ``delta`` (may be None) into
                    the 32-bit residual ``h`` in place and returns the normed rows in
                    the activation dtype; with ``rows`` it returns the norm of the
                    picked rows of ``h + delta`` and leaves ``h`` alone.
``PositionEncoding````tables()``: what the mixer's kernels need to place a token.
``Mixer``           ``cache_need()``: a :class:`KVCacheNeed`, a :class:`StateNeed`
                    or None; ``forward(x, step, cache)`` mixes tokens of the same
                    request, reading and writing only its own cache.
``FeedForward``     ``forward(x)``: works on each token alone.
``Block``           ``mixer`` attribute and ``forward(h, pending, step, cache)``:
                    arranges norms, mixer, feed-forward and residual sums; returns
                    the update not yet added into ``h``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch

from ..config.spec import PartSpec


# ------------------------------------------------------------------ declarations
@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part needs.  ``init`` says how the random-weights mode fills it:
    ``matrix`` normal(0, 0.02), ``norm`` 1 + U(-0.1, 0.1), ``zeros``; ``integer``
    tensors are kept as int32, others in the run's dtype (bfloat16 or float32)
    unless the file stores them in 32-bit, in which case they stay so."""

    shape: tuple[int, ...]
    init: str = "matrix"
    optional: bool = False
    integer: bool = False


@dataclass(frozen=True)
class KVCacheNeed:
    """Keys and values per token in pages.  ``window`` None: every earlier key stays
    visible; an integer w: a query at position i reads keys i-w+1 .. i, and pages
    wholly behind that may be given back."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request (zero when the request starts)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class BuildContext:
    """What a part may use while it is built."""

    device: torch.device
    dtype: torch.dtype                      # activations and matrices: float32 or bfloat16
    max_positions: int                      # the engine's limit on a request's length
    shared: dict = field(default_factory=dict)   # tables shared by equal parts (rotary tables)


class Part:
    def __init__(self, params: dict[str, Any], ctx: BuildContext):
        self.params = params
        self.ctx = ctx

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receives the device tensors named in :meth:`tensor_specs`."""


class Norm(Part):
    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Mixer(Part):
    # True if forward() only launches kernels that read the step's device arrays (no
    # host-side loop over requests, no synchronisation): decode steps of a model whose
    # mixers all say so are replayed from CUDA graphs.
    graph_safe = False

    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], step, cache) -> Optional[torch.Tensor]:
        raise NotImplementedError


# ---------------------------------------------------------------------- registry
_PARTS: dict[str, Callable[[dict, BuildContext], Part]] = {}


def register_part(kind: str, factory: Callable[[dict, BuildContext], Part], *, replace: bool = False) -> None:
    if kind in _PARTS and not replace:
        raise ValueError(f"part kind {kind!r} is already registered")
    _PARTS[kind] = factory


def unregister_part(kind: str) -> None:
    _PARTS.pop(kind, None)


def make_part(spec: PartSpec, ctx: BuildContext) -> Part:
    if spec.kind not in _PARTS:
        raise KeyError(f"no part of kind {spec.kind!r}; registered: {', '.join(sorted(_PARTS))}")
    return _PARTS[spec.kind](dict(spec.params), ctx)


def prefixed(prefix: str, specs: dict[str, TensorSpec]) -> dict[str, TensorSpec]:
    return {prefix + k: v for k, v in specs.items()}


def take(tensors: dict[str, torch.Tensor], prefix: str) -> dict[str, torch.Tensor]:
    """The tensors under ``prefix``, with the prefix removed."""
    n = len(prefix)
    return {k[n:]: v for k, v in tensors.items() if k.startswith(prefix)}
