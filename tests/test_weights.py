"""Weights: the safetensors reader/writer, the one error that lists everything wrong, kept
precisions, the random-weights mode."""

import json
import struct

import pytest
import torch

from clockwork_b200.config import spec_from_raw
from clockwork_b200.parts import build_model
from clockwork_b200.weights import (
    CheckpointIndex, SafetensorsError, SafetensorsFile, WeightMismatchError, load_checkpoint_into,
    save_safetensors, write_random_model,
)
from clockwork_b200.weights.loader import kept_dtype
from tests.plain.qwen2_plain import read_model_dir
from tests.tiny_configs import TINY_A, TINY_B


def test_safetensors_round_trip(tmp_path):
    tensors = {
        "a": torch.arange(12, dtype=torch.float32).reshape(3, 4),
        "b": torch.randn(5).to(torch.bfloat16),
        "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
    }
    save_safetensors(tmp_path / "m.safetensors", tensors, {"k": "v"})
    f = SafetensorsFile(tmp_path / "m.safetensors")
    assert f.metadata == {"k": "v"}
    for name, t in tensors.items():
        got = f.tensor(name)
        assert got.dtype == t.dtype and torch.equal(got, t)
    # the independent reader of the plain implementation agrees
    (tmp_path / "config.json").write_text("{}")
    save_safetensors(tmp_path / "model.safetensors", tensors)
    _, plain = read_model_dir(tmp_path, dtype=torch.float32)
    assert torch.equal(plain["a"], tensors["a"]) and torch.equal(plain["b"], tensors["b"].float())


def test_truncated_and_malformed_files(tmp_path):
    path = tmp_path / "m.safetensors"
    save_safetensors(path, {"a": torch.zeros(100)})
    blob = path.read_bytes()
    path.write_bytes(blob[:-40])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(path)
    path.write_bytes(blob[:5])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(path)
    path.write_bytes(struct.pack("<Q", 10**9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(path)
    with pytest.raises(FileNotFoundError, match="no .safetensors"):
        CheckpointIndex(tmp_path / "nothing")


def test_random_model_is_deterministic_and_distributed(tmp_path):
    a1 = write_random_model(tmp_path / "a1", TINY_A, seed=0)
    a2 = write_random_model(tmp_path / "a2", TINY_A, seed=0)
    a3 = write_random_model(tmp_path / "a3", TINY_A, seed=1)
    assert (a1 / "model.safetensors").read_bytes() == (a2 / "model.safetensors").read_bytes()
    assert (a1 / "model.safetensors").read_bytes() != (a3 / "model.safetensors").read_bytes()
    assert json.loads((a1 / "config.json").read_text())["hidden_size"] == 64
    _, w = read_model_dir(a1)
    assert "lm_head.weight" not in w  # tied
    emb, norm = w["model.embed_tokens.weight"], w["model.layers.0.input_layernorm.weight"]
    assert abs(float(emb.std()) - 0.02) < 0.002 and abs(float(emb.mean())) < 0.002
    assert abs(float(norm.mean()) - 1.0) < 0.05 and 0.05 < float(norm.std()) < 0.15
    _, wb = read_model_dir(write_random_model(tmp_path / "b", TINY_B, seed=1))
    assert wb["lm_head.weight"].shape == (320, 96) and wb["model.layers.2.mlp.gate_proj.weight"].shape == (200, 96)
    assert wb["model.layers.0.self_attn.k_proj.bias"].shape == (32,)


def _model(raw):
    return build_model(spec_from_raw(raw), torch.float32, "cpu")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(tmp_path / "m", TINY_B, seed=1)
    _, w = read_model_dir(folder, dtype=torch.float32)
    w.pop("model.layers.1.mlp.up_proj.weight")
    w.pop("model.norm.weight")
    w["model.layers.9.extra"] = torch.zeros(3)
    w["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(7)
    save_safetensors(folder / "model.safetensors", w)
    with pytest.raises(WeightMismatchError) as info:
        load_checkpoint_into(_model(TINY_B), folder)
    err = info.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra"]
    assert [n for n, _, _ in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.bias"]
    text = str(err)
    assert "missing=" in text and "unexpected=" in text and "[7] != model [96]" in text


def test_tied_head_may_be_absent_untied_may_not(tmp_path):
    folder = write_random_model(tmp_path / "a", TINY_A, seed=0)
    load_checkpoint_into(_model(TINY_A), folder)  # no lm_head.weight in the file: fine when tied
    folder_b = write_random_model(tmp_path / "b", TINY_B, seed=1)
    _, w = read_model_dir(folder_b, dtype=torch.float32)
    w.pop("lm_head.weight")
    save_safetensors(folder_b / "model.safetensors", w)
    with pytest.raises(WeightMismatchError, match="lm_head.weight"):
        load_checkpoint_into(_model(TINY_B), folder_b)


def test_kept_precisions(tmp_path):
    assert kept_dtype("matrix", torch.bfloat16) == torch.bfloat16 and kept_dtype("table", torch.float32) == torch.float32
    assert kept_dtype("vector", torch.bfloat16) == torch.float32 and kept_dtype("state32", torch.bfloat16) == torch.float32
    assert kept_dtype("index", torch.bfloat16) == torch.int32
    folder = write_random_model(tmp_path / "a", TINY_A, seed=0)
    model = build_model(spec_from_raw(TINY_A), torch.bfloat16, "cpu")
    load_checkpoint_into(model, folder)
    attn = model.blocks[0].mixer
    assert attn.qkv.weight.dtype == torch.bfloat16 and attn.qkv.weight.shape == (128, 64)
    assert attn.qkv.bias.dtype == torch.float32 and model.final_norm.weight.dtype == torch.float32
    assert model.head.weight.data_ptr() == model.embedding.data_ptr()  # tied
    # q, k and v rows were concatenated in that order
    _, w = read_model_dir(folder, dtype=torch.float32)
    want = torch.cat([w[f"model.layers.0.self_attn.{p}_proj.weight"] for p in "qkv"])
    assert torch.equal(attn.qkv.weight.float(), want)
