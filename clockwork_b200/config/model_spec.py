"""Architecture-neutral description of a model: what each layer is made of, and in which
order layers run.

An architecture (``clockwork_b200/models``) turns its own ``config.json`` keys into one
``ModelSpec``.  Everything below the spec (parts, cache manager, step function) reads sizes
and constants from the spec only, so no part knows which model it is in.

A spec is plain data:

* ``layers[i]`` names the mixer, feed-forward, norms and block arrangement of layer ``i``
  by *kind* strings that the part registry (``clockwork_b200/parts/registry.py``) resolves.
  Different layers may use different kinds and sizes.
* ``schedule`` is the order in which layers run.  An entry may name a layer twice, or let
  a layer read the cache that another layer wrote (``cache_layer`` differs from ``layer``
  and ``write_cache`` is false).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """A part kind plus its parameters (sizes, constants, flags)."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict, hash=False)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer, a feed-forward and their norms."""

    block: str  # block arrangement kind, e.g. "prenorm_residual"
    mixer: PartSpec
    ffn: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    prefix: str  # checkpoint name prefix of the layer's tensors, e.g. "model.layers.3"


@dataclass(frozen=True)
class ExecStep:
    """One entry of the run order."""

    layer: int  # index into ModelSpec.layers (whose weights run)
    cache_layer: int | None = None  # cache written/read; None means ``layer``
    write_cache: bool = True  # False: read what ``cache_layer`` already holds for these tokens

    def resolved_cache_layer(self) -> int:
        return self.layer if self.cache_layer is None else self.cache_layer


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: list[LayerSpec]
    schedule: list[ExecStep]
    final_norm: PartSpec
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm"
    head_name: str = "lm_head.weight"
    tie_word_embeddings: bool = False
    eos_token_ids: tuple[int, ...] = ()
    max_position_embeddings: int | None = None
    raw: dict[str, Any] = field(default_factory=dict)  # the config.json it came from

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ValueError("vocab_size and hidden_size must be positive")
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        writers: set[int] = set()
        for step in self.schedule:
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"schedule names layer {step.layer}, model has {len(self.layers)}")
            cache_layer = step.resolved_cache_layer()
            if not 0 <= cache_layer < len(self.layers):
                raise ValueError(f"schedule names cache layer {cache_layer}")
            if step.write_cache:
                writers.add(cache_layer)
            elif cache_layer not in writers:
                raise ValueError(
                    f"layer {step.layer} reads cache layer {cache_layer} before any layer wrote it"
                )


def sequential_schedule(num_layers: int) -> list[ExecStep]:
    return [ExecStep(layer=i) for i in range(num_layers)]
