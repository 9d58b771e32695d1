"""Random-weights mode: draw every declared tensor from a seed and write a model folder
(``config.json`` + ``model.safetensors``), or fill a model on the device without a file.

Distributions: linear weights, biases and embeddings N(0, 0.02); norm weights 1 + N(0, 0.1).
The reference's counterpart builds a Hugging Face model under ``torch.manual_seed``
(``clockwork/engine/loader.py:82-103``); here each tensor is drawn from its own generator
seeded by (seed, tensor name), so a tensor's values do not depend on which other tensors
exist or on the order of drawing.
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Any, Iterable

import numpy as np
import torch

from .decl import TensorDecl
from .safetensors_io import save_safetensors

_STORE_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _generator(seed: int, name: str) -> np.random.Generator:
    return np.random.default_rng(np.random.SeedSequence([int(seed), zlib.crc32(name.encode("utf-8"))]))


def draw_tensor(decl: TensorDecl, seed: int) -> torch.Tensor:
    """float32 (or int32) CPU tensor for one declaration."""
    rng = _generator(seed, decl.name)
    if decl.init == "index":
        n = int(np.prod(decl.shape))
        return torch.arange(n, dtype=torch.int32).reshape(decl.shape)
    if decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=torch.float32)
    values = rng.standard_normal(size=decl.shape, dtype=np.float32)
    if decl.init == "norm":
        values = np.float32(1.0) + np.float32(0.1) * values
    else:  # linear, bias, embedding
        values = np.float32(0.02) * values
    return torch.from_numpy(values)


def write_random_model(
    out_dir: str | Path,
    config_json: dict[str, Any],
    seed: int = 0,
    store_dtype: str = "bfloat16",
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for the architecture that
    ``config_json`` names.  Matrices and tables are stored in ``store_dtype``; vectors
    (norm weights, biases) likewise, so that both run precisions read identical values."""
    from ..config.registry import spec_from_raw
    from ..parts.model import tensor_decls_for_spec

    if store_dtype not in _STORE_DTYPES:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE_DTYPES)}")
    spec = spec_from_raw(config_json)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    tensors: dict[str, torch.Tensor] = {}
    for decl in tensor_decls_for_spec(spec):
        if decl.optional:
            continue
        t = draw_tensor(decl, seed)
        if t.dtype == torch.float32 and decl.role != "state32":
            t = t.to(_STORE_DTYPES[store_dtype])
        tensors[decl.name] = t
    (out / "config.json").write_text(json.dumps(config_json, indent=2) + "\n", encoding="utf-8")
    save_safetensors(out / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return out


def fill_model_on_device(model, seed: int = 0) -> None:
    """Fill ``model`` with random weights drawn on its device (no file, no host copy):
    for models whose weights would take long to draw on the host.  Same distributions as
    ``write_random_model``, different values."""
    decls: Iterable[TensorDecl] = model.tensor_decls()
    by_name = {d.name: d for d in decls}
    from .loader import kept_dtype

    def fetch(name: str) -> torch.Tensor:
        decl = by_name[name]
        gen = torch.Generator(device=model.device)
        gen.manual_seed((int(seed) << 32) ^ zlib.crc32(name.encode("utf-8")))
        dtype = kept_dtype(decl.role, model.dtype)
        if decl.init == "index":
            return torch.arange(int(np.prod(decl.shape)), dtype=torch.int32, device=model.device).reshape(decl.shape)
        if decl.init == "zeros":
            return torch.zeros(decl.shape, dtype=dtype, device=model.device)
        t = torch.empty(decl.shape, dtype=torch.float32, device=model.device)
        t.normal_(0.0, 1.0, generator=gen)
        if decl.init == "norm":
            t.mul_(0.1).add_(1.0)
        else:
            t.mul_(0.02)
        return t.to(dtype)

    model.load_weights(fetch)
