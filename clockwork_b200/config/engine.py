"""Engine configuration: model, cache and scheduler sections, YAML files and flat overrides.

The field names and meanings follow the reference's ``clockwork/config.py:17-87``
(``ModelConfig``, ``CacheConfig``, ``SchedulerConfig``, ``EngineConfig``) so that its
YAML profiles load unchanged.  Fields that only made sense for a multi-backend
engine (``device``, ``trust_remote_code``, ``attention_backend``) are accepted in a
YAML file and ignored; new fields are ``prefill_chunk_size`` (the scheduler cuts
prompts into portions, which the reference does not) and ``num_state_slots``.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from pathlib import Path

import yaml

DTYPES = ("float32", "bfloat16")
# accepted on input for compatibility with the reference's profiles, mapped to bfloat16
_DTYPE_ALIASES = {"float16": "bfloat16", "bf16": "bfloat16", "fp32": "float32"}
_IGNORED_MODEL_KEYS = ("device", "trust_remote_code")


def normalise_dtype(name: str) -> str:
    name = _DTYPE_ALIASES.get(name, name)
    if name not in DTYPES:
        raise ValueError(f"unknown dtype {name!r}, expected one of {DTYPES}")
    return name


@dataclass
class ModelConfig:
    """Which model folder to serve and in which precision (reference ``config.py:17-31``)."""

    model: str
    dtype: str = "bfloat16"
    max_model_len: int = 4096
    seed: int = 0
    cuda_graphs: bool = True  # replay captured graphs for steps in which every request decodes one token

    def __post_init__(self) -> None:
        self.dtype = normalise_dtype(self.dtype)


@dataclass
class CacheConfig:
    """Page pool geometry (reference ``config.py:34-39``)."""

    block_size: int = 16
    num_blocks: int = 512
    enable_prefix_cache: bool = True
    watermark: float = 0.01
    num_state_slots: int | None = None  # default: scheduler.max_num_seqs


@dataclass
class SchedulerConfig:
    """Batching limits (reference ``config.py:42-47``)."""

    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    max_model_len: int = 4096
    preemption_mode: str = "recompute"
    prefill_chunk_size: int | None = None  # None: a portion may use the whole token budget

    def __post_init__(self) -> None:
        if self.preemption_mode != "recompute":
            raise ValueError(
                f"preemption_mode {self.preemption_mode!r} is not supported; only 'recompute' exists"
            )


def _section(cls, data: dict | None, where: str, ignored: tuple[str, ...] = ()):
    data = dict(data or {})
    for key in ignored:
        data.pop(key, None)
    known = {f.name for f in fields(cls)}
    unknown = sorted(set(data) - known)
    if unknown:
        raise ValueError(f"{where}: unknown keys {unknown}; known keys are {sorted(known)}")
    return cls(**data)


@dataclass
class EngineConfig:
    model: ModelConfig
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)

    @classmethod
    def from_yaml(cls, path: str | Path) -> "EngineConfig":
        """Load a profile; a top-level ``model:`` section with a ``model:`` key is required
        (reference ``config.py:57-68``)."""
        data = yaml.safe_load(Path(path).read_text(encoding="utf-8")) or {}
        model = data.get("model")
        if not isinstance(model, dict) or "model" not in model:
            raise ValueError(f"{path}: expected a top-level 'model' section naming the model")
        extra = sorted(set(data) - {"model", "cache", "scheduler", "attention_backend"})
        if extra:
            raise ValueError(f"{path}: unknown top-level sections {extra}")
        return cls(
            model=_section(ModelConfig, model, f"{path}: model", _IGNORED_MODEL_KEYS),
            cache=_section(CacheConfig, data.get("cache"), f"{path}: cache"),
            scheduler=_section(SchedulerConfig, data.get("scheduler"), f"{path}: scheduler"),
        )

    @classmethod
    def defaults(cls, model: str, **overrides) -> "EngineConfig":
        """Defaults plus flat overrides; a key is set on every section that has it
        (``max_model_len`` lands on model and scheduler), an unknown key is an error
        (reference ``config.py:70-87``)."""
        cfg = cls(model=ModelConfig(model=model))
        cfg.apply_overrides(overrides)
        return cfg

    def apply_overrides(self, overrides: dict) -> None:
        for key, value in overrides.items():
            targets = [
                sub
                for sub in (self.model, self.cache, self.scheduler)
                if key in {f.name for f in fields(sub)}
            ]
            if not targets:
                raise ValueError(f"unknown config override {key!r}")
            for sub in targets:
                setattr(sub, key, value)
        self.model.dtype = normalise_dtype(self.model.dtype)

    def apply_pairs(self, pairs: list[str]) -> None:
        """``KEY=VALUE`` strings as the reference's ``scripts/serve.py:13-30`` takes with ``--set``."""
        parsed = {}
        for pair in pairs:
            if "=" not in pair:
                raise ValueError(f"override {pair!r} is not KEY=VALUE")
            key, raw = pair.split("=", 1)
            parsed[key] = yaml.safe_load(raw)
        self.apply_overrides(parsed)
