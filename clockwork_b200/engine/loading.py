"""From a model folder (or a description plus a seed) to a model with weights on the device."""

from __future__ import annotations

from pathlib import Path

import torch

from .. import models  # noqa: F401  (registers architectures)
from ..config.registry import spec_from_dir, spec_from_raw
from ..parts.model import DecoderModel, build_model
from ..weights.loader import load_checkpoint_into
from ..weights.random_init import fill_model_on_device

TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def run_dtype(name: str) -> torch.dtype:
    from ..config.engine import normalise_dtype

    return TORCH_DTYPES[normalise_dtype(name)]


def load_model(model_dir: str | Path, dtype: str = "bfloat16", device: str = "cuda:0") -> DecoderModel:
    """The model class is chosen by ``config.json``'s architecture name; weights come from the
    folder's safetensors by tensor name."""
    spec = spec_from_dir(model_dir)
    model = build_model(spec, run_dtype(dtype), device)
    load_checkpoint_into(model, model_dir)
    return model


def random_model(config_json: dict, seed: int = 0, dtype: str = "bfloat16", device: str = "cuda:0") -> DecoderModel:
    """A model of the described architecture with random weights drawn on the device."""
    spec = spec_from_raw(config_json)
    model = build_model(spec, run_dtype(dtype), device)
    fill_model_on_device(model, seed)
    return model
