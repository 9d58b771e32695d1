"""Configuration: engine profiles, flat overrides, config.json parsing, the architecture registry."""

import json

import pytest

from clockwork_b200.config import EngineConfig, registered_architectures, spec_from_raw
from clockwork_b200.models import Qwen2Config
from tests.tiny_configs import TINY_A, TINY_B


def test_defaults_and_overrides_route_to_every_section():
    cfg = EngineConfig.defaults("m", max_model_len=128, num_blocks=7, max_num_seqs=3, dtype="float32")
    assert cfg.model.max_model_len == 128 and cfg.scheduler.max_model_len == 128
    assert cfg.cache.num_blocks == 7 and cfg.scheduler.max_num_seqs == 3 and cfg.model.dtype == "float32"
    with pytest.raises(ValueError, match="unknown config override"):
        EngineConfig.defaults("m", no_such_key=1)


def test_yaml_profile_and_pairs(tmp_path):
    path = tmp_path / "p.yaml"
    path.write_text("model:\n  model: /x\n  dtype: float32\n  device: cuda\ncache:\n  block_size: 8\nscheduler:\n  max_num_seqs: 5\nattention_backend: auto\n")
    cfg = EngineConfig.from_yaml(path)
    assert cfg.model.model == "/x" and cfg.cache.block_size == 8 and cfg.scheduler.max_num_seqs == 5
    cfg.apply_pairs(["num_blocks=33", "watermark=0.5", "prefill_chunk_size=7"])
    assert cfg.cache.num_blocks == 33 and cfg.cache.watermark == 0.5 and cfg.scheduler.prefill_chunk_size == 7
    with pytest.raises(ValueError, match="KEY=VALUE"):
        cfg.apply_pairs(["oops"])
    bad = tmp_path / "bad.yaml"
    bad.write_text("cache:\n  block_size: 8\n")
    with pytest.raises(ValueError, match="top-level 'model' section"):
        EngineConfig.from_yaml(bad)
    bad.write_text("model:\n  model: /x\ncache:\n  blok_size: 8\n")
    with pytest.raises(ValueError, match="unknown keys"):
        EngineConfig.from_yaml(bad)


def test_reference_profiles_load():
    import pathlib

    from tests.tiny_configs import reference_checkout

    ref = pathlib.Path(reference_checkout(), "configs")
    if not ref.is_dir():
        pytest.skip("reference checkout not present")
    for path in ref.glob("*.yaml"):
        cfg = EngineConfig.from_yaml(path)
        assert cfg.cache.block_size == 16


def test_dtype_whitelist():
    with pytest.raises(ValueError, match="unknown dtype"):
        EngineConfig.defaults("m", dtype="int8")


def test_qwen2_config_reads_every_key():
    a, b = Qwen2Config.from_raw(TINY_A), Qwen2Config.from_raw(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 3, 1, 32)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.rms_norm_eps == 1e-6 and b.rms_norm_eps == 1e-5 and a.rope_theta == 1e4 and b.rope_theta == 1e6
    raw = dict(TINY_A)
    del raw["head_dim"]
    assert Qwen2Config.from_raw(raw).head_dim == 16  # hidden_size // num_attention_heads
    raw = dict(TINY_A, rope_parameters={"rope_type": "default", "rope_theta": 5.0})
    assert Qwen2Config.from_raw(raw).rope_theta == 5.0
    raw = dict(TINY_A, eos_token_id=[3, 4])
    assert Qwen2Config.from_raw(raw).eos_token_ids == (3, 4)


@pytest.mark.parametrize("change, error", [
    ({"hidden_act": "gelu"}, NotImplementedError),
    ({"use_sliding_window": True}, NotImplementedError),
    ({"model_type": "llama"}, ValueError),
    ({"num_key_value_heads": 3}, ValueError),
    ({"rope_parameters": {"rope_type": "yarn", "rope_theta": 1.0}}, NotImplementedError),
    ({"vocab_size": None}, ValueError),
    ({"rms_norm_eps": "x"}, ValueError),
])
def test_qwen2_config_rejects(change, error):
    with pytest.raises(error):
        Qwen2Config.from_raw(dict(TINY_A, **change))


def test_registry_and_spec():
    assert "Qwen2ForCausalLM" in registered_architectures()
    spec = spec_from_raw(TINY_B)
    assert len(spec.layers) == 3 and [s.layer for s in spec.schedule] == [0, 1, 2]
    mixer = spec.layers[0].mixer
    assert mixer.kind == "attention" and mixer["num_heads"] == 3 and mixer["qkv_bias"] and not mixer["o_bias"]
    assert mixer["position"].kind == "rope_neox" and mixer["position"]["theta"] == 1e6
    assert spec.layers[1].ffn["intermediate_size"] == 200 and spec.final_norm["eps"] == 1e-5
    with pytest.raises(ValueError, match="unknown architecture.*Qwen2ForCausalLM"):
        spec_from_raw(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ValueError, match="exactly one architecture"):
        spec_from_raw({k: v for k, v in TINY_A.items() if k != "architectures"})
    # the description survives a round trip through config.json text
    assert spec_from_raw(json.loads(json.dumps(spec.raw))).layers[0].mixer.params["head_dim"] == 32


def test_schedule_validation():
    from clockwork_b200.config import ExecStep

    spec = spec_from_raw(TINY_A)
    spec.schedule = [ExecStep(0), ExecStep(1, cache_layer=0, write_cache=False), ExecStep(0)]
    spec.validate()
    spec.schedule = [ExecStep(1, cache_layer=0, write_cache=False)]
    with pytest.raises(ValueError, match="before any layer wrote it"):
        spec.validate()
    spec.schedule = [ExecStep(5)]
    with pytest.raises(ValueError, match="names layer 5"):
        spec.validate()
