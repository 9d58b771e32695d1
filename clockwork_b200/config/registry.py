"""One registry from an architecture's name (``config.json["architectures"][0]``) to the
object that reads its configuration and describes its model.

The reference has no registry: its loader hard-checks ``model_type == "qwen2"``
(``clockwork/engine/loader.py:69-71``).  Here an architecture is any object with

    name: str
    def parse_config(self, raw: dict) -> TypedConfig      # validates config.json keys
    def model_spec(self, config: TypedConfig) -> ModelSpec

registered under its name.  Everything else in the framework goes through ``ModelSpec``.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Protocol

from .model_spec import ModelSpec


class Architecture(Protocol):
    name: str

    def parse_config(self, raw: dict[str, Any]) -> Any: ...

    def model_spec(self, config: Any) -> ModelSpec: ...


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    return arch


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ValueError(
            f"unknown architecture {name!r}; registered architectures: {registered_architectures()}"
        ) from None


def named_shapes() -> dict[str, dict[str, Any]]:
    """Every size that a registered architecture knows by name (its optional ``named_shapes``
    attribute): name -> config.json contents, the architecture's own name inside."""
    out: dict[str, dict[str, Any]] = {}
    for arch in _ARCHITECTURES.values():
        out.update(getattr(arch, "named_shapes", {}))
    return out


def shape_config(name: str, num_layers: int | None = None) -> dict[str, Any]:
    """The config.json of a named size, optionally with fewer (or more) layers."""
    shapes = named_shapes()
    if name not in shapes:
        raise ValueError(f"unknown shape {name!r}; known: {sorted(shapes)}")
    raw = dict(shapes[name])
    if num_layers is not None:
        arch = get_architecture(architecture_name(raw))
        raw[getattr(arch, "layer_count_key", "num_hidden_layers")] = num_layers
    return raw


def architecture_name(raw: dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ValueError(
            "config.json must name exactly one architecture in 'architectures', "
            f"got {archs!r}; registered architectures: {registered_architectures()}"
        )
    return archs[0]


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and *.safetensors")
    return json.loads(path.read_text(encoding="utf-8"))


def spec_from_raw(raw: dict[str, Any]) -> ModelSpec:
    arch = get_architecture(architecture_name(raw))
    spec = arch.model_spec(arch.parse_config(raw))
    spec.validate()
    return spec


def spec_from_dir(model_dir: str | Path) -> ModelSpec:
    return spec_from_raw(read_config_json(model_dir))
