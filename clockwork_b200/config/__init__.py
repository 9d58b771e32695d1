from .engine import CacheConfig, EngineConfig, ModelConfig, SchedulerConfig, normalise_dtype
from .model_spec import ExecStep, LayerSpec, ModelSpec, PartSpec, sequential_schedule
from .registry import (
    architecture_name,
    get_architecture,
    read_config_json,
    register_architecture,
    registered_architectures,
    spec_from_dir,
    spec_from_raw,
)

__all__ = [
    "CacheConfig", "EngineConfig", "ModelConfig", "SchedulerConfig", "normalise_dtype",
    "ExecStep", "LayerSpec", "ModelSpec", "PartSpec", "sequential_schedule",
    "architecture_name", "get_architecture", "read_config_json", "register_architecture",
    "registered_architectures", "spec_from_dir", "spec_from_raw",
]
