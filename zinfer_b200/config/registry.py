"""The one registry from an architecture's name to its model.

An entry holds the typed configuration class and the function that turns a
configuration into a :class:`ModelSpec`.  Lookup is by ``architectures[0]`` of
config.json, with ``model_type`` as a second key; the reference detects the family
by ``model_type`` alone (src/model/runtime/decoder_family.zig:267-281) and keeps
its entries in a table of constants and functions
(src/model/runtime/decoder_registry.zig:7-21).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable

from .spec import ModelSpec


@dataclass(frozen=True)
class Family:
    name: str
    model_type: str
    config_class: Any                          # has from_dict(dict) and to_dict()
    model_spec: Callable[[Any], ModelSpec]     # configuration -> what to build


_FAMILIES: dict[str, Family] = {}


class UnknownArchitecture(ValueError):
    pass


def register_family(family: Family, *, replace: bool = False) -> None:
    for key in (family.name, family.model_type):
        if key in _FAMILIES and not replace and _FAMILIES[key] is not family:
            raise ValueError(f"architecture key {key!r} is already registered")
        _FAMILIES[key] = family


def unregister_family(name: str) -> None:
    fam = _FAMILIES.pop(name, None)
    if fam is not None:
        for key in (fam.name, fam.model_type):
            _FAMILIES.pop(key, None)


def registered() -> list[str]:
    return sorted({f.name for f in _FAMILIES.values()})


def family_for(config: dict) -> Family:
    """Family of a raw config.json dictionary."""
    keys = list(config.get("architectures") or [])[:1]
    if "model_type" in config:
        keys.append(config["model_type"])
    if not keys:
        raise UnknownArchitecture("config.json names neither `architectures` nor `model_type`")
    for k in keys:
        if k in _FAMILIES:
            return _FAMILIES[k]
    raise UnknownArchitecture(
        f"no model registered for {' / '.join(map(repr, keys))}; registered: {', '.join(registered()) or 'none'}")


def load_config(model_dir: str) -> tuple[Family, Any]:
    """(family, typed configuration) of a model folder."""
    path = os.path.join(model_dir, "config.json")
    with open(path) as f:
        raw = json.load(f)
    fam = family_for(raw)
    return fam, fam.config_class.from_dict(raw)
