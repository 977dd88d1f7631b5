"""Architecture-independent description of a decoder: what the engine builds from.

An architecture's typed configuration (for example :class:`Qwen3Config`) is turned
into a :class:`ModelSpec` by its family function.  The spec names parts by ``kind``
and gives every size and constant as a parameter, layer by layer, so one model may
use different mixers and feed-forwards in different layers.  The order in which
layers run is data as well: ``schedule`` is a list of :class:`ScheduleEntry`, which
may name a layer twice, and an entry may read the cache another entry wrote.

The reference keeps the same split between constants and code with its
``Spec``/``LayerLayout`` structs (src/model/layers/rmsnorm_gqa_swiglu_block.zig:10-51).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by ``kind`` from the parts registry, with its parameters."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:  # params hold only scalars and nested PartSpecs
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward.

    ``prefix`` is prepended to the tensor names the parts declare
    (``model.layers.3.`` for layer 3 of Qwen3, src/model/families/qwen3/weights.zig:10-19).
    """

    block: PartSpec
    prefix: str


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers``.  ``cache`` names the cache this run
    uses; entries with the same ``cache`` share it, the first of them in schedule
    order writes it and the later ones only read it.  ``None`` gives the entry a
    cache of its own.
    """

    layer: int
    cache: Optional[str] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple[int, ...] = ()

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("ModelSpec has no layers")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {e.layer}, but there are {len(self.layers)} layers")


def default_schedule(n_layers: int) -> tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i) for i in range(n_layers))
