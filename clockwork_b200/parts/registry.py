"""Part kinds by name.  A model description names kinds; this is where they resolve to classes.
New kinds are added with the ``register_*`` functions, from inside or outside the package."""

from __future__ import annotations

from typing import Callable

import torch

from ..config.model_spec import LayerSpec, PartSpec

_KINDS: dict[str, dict[str, Callable]] = {"norm": {}, "position": {}, "mixer": {}, "ffn": {}, "block": {}}


def _register(category: str, kind: str, cls, replace: bool) -> None:
    table = _KINDS[category]
    if kind in table and not replace:
        raise ValueError(f"{category} kind {kind!r} is already registered")
    table[kind] = cls


def register_norm(kind: str, cls, *, replace: bool = False) -> None:
    _register("norm", kind, cls, replace)


def register_position(kind: str, cls, *, replace: bool = False) -> None:
    _register("position", kind, cls, replace)


def register_mixer(kind: str, cls, *, replace: bool = False) -> None:
    _register("mixer", kind, cls, replace)


def register_ffn(kind: str, cls, *, replace: bool = False) -> None:
    _register("ffn", kind, cls, replace)


def register_block(kind: str, cls, *, replace: bool = False) -> None:
    _register("block", kind, cls, replace)


def registered(category: str) -> list[str]:
    return sorted(_KINDS[category])


def build_part(category: str, spec: PartSpec, prefix: str, dtype: torch.dtype, device):
    table = _KINDS[category]
    if spec.kind not in table:
        raise ValueError(f"unknown {category} kind {spec.kind!r}; registered: {sorted(table)}")
    return table[spec.kind](spec, prefix, dtype, torch.device(device))


def build_block(layer: LayerSpec, dtype: torch.dtype, device):
    table = _KINDS["block"]
    if layer.block not in table:
        raise ValueError(f"unknown block kind {layer.block!r}; registered: {sorted(table)}")
    return table[layer.block](layer, dtype, torch.device(device))
