"""Shared fixtures.  Tests marked ``gpu`` need a CUDA device; everything else runs on the CPU."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from tests.tiny_configs import TINY  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """{name: model folder} of the tiny random models, written once per session to a temp folder."""
    from clockwork_b200.weights import write_random_model

    out = {}
    for name, (raw, seed, _page) in TINY.items():
        out[name] = write_random_model(tmp_path_factory.mktemp(f"tiny_{name}"), raw, seed=seed)
    return out


@pytest.fixture(scope="session")
def sharp_dirs(tmp_path_factory, tiny_dirs):
    """The tiny models with q and k projections scaled up so that attention is peaked: with the
    default N(0, 0.02) weights every softmax is nearly uniform and a missed or misplaced key
    would change the output by less than the tolerance."""
    import json

    from clockwork_b200.weights import save_safetensors
    from tests.plain.qwen2_plain import read_model_dir

    out = {}
    for name, folder in tiny_dirs.items():
        config, weights = read_model_dir(folder, dtype=torch.float32)
        scaled = {}
        for key, w in weights.items():
            if ".q_proj." in key or ".k_proj." in key:
                w = w * 12.0
            scaled[key] = w.to(torch.bfloat16)
        target = tmp_path_factory.mktemp(f"sharp_{name}")
        (target / "config.json").write_text(json.dumps(config))
        save_safetensors(target / "model.safetensors", scaled)
        out[name] = target
    return out
