"""Qwen2 / Qwen2.5 dense decoder: its config.json keys and its model description.

Follows the reference's ``clockwork/engine/model.py``: pre-norm RMSNorm blocks
(``model.py:131-154``), grouped-query attention with biased q/k/v and bias-free o
projections (``model.py:74-77``), rotate-half rotary position encoding at ``rope_theta``
(``model.py:21-35``, ``171-191``), a SwiGLU feed-forward (``model.py:52-63``), full causal
attention (``model.py:211-212`` rejects sliding windows) and a tied or untied output head
(``model.py:216-218``).  Tensor names are the Hugging Face names the reference loads
unchanged (``clockwork/engine/loader.py:57-64``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ..config.model_spec import LayerSpec, ModelSpec, PartSpec, sequential_schedule
from ..config.registry import register_architecture


def _require(raw: dict[str, Any], key: str, kind):
    if key not in raw or raw[key] is None:
        raise ValueError(f"config.json: missing required key {key!r}")
    value = raw[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ValueError(f"config.json: {key!r} must be an integer, got {value!r}")
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ValueError(f"config.json: {key!r} must be a number, got {value!r}")
        value = float(value)
    return value


@dataclass(frozen=True)
class Qwen2Config:
    """Typed view of a Qwen2 ``config.json`` (keys as the reference reads them)."""

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...]
    max_position_embeddings: int | None

    @classmethod
    def from_raw(cls, raw: dict[str, Any]) -> "Qwen2Config":
        model_type = raw.get("model_type", "qwen2")
        if model_type != "qwen2":  # clockwork/engine/loader.py:70-71
            raise ValueError(f"expected a qwen2 model, got model_type={model_type!r}")
        hidden_act = raw.get("hidden_act", "silu")
        if hidden_act != "silu":  # clockwork/engine/model.py:55-57
            raise NotImplementedError(f"hidden_act {hidden_act!r} is not supported")
        if raw.get("use_sliding_window", False):  # clockwork/engine/model.py:211-212
            raise NotImplementedError("sliding-window attention is not supported")
        hidden = _require(raw, "hidden_size", int)
        heads = _require(raw, "num_attention_heads", int)
        kv_heads = _require(raw, "num_key_value_heads", int)
        head_dim = raw.get("head_dim") or hidden // heads  # clockwork/engine/model.py:17-18
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads != 0:
            # clockwork/kernels/attention.py:39-40
            raise ValueError(f"num_heads {heads} not a multiple of num_kv_heads {kv_heads}")
        if head_dim <= 0 or head_dim % 2 != 0:
            raise ValueError(f"head_dim {head_dim} must be positive and even for rotate-half RoPE")
        # transformers 5.x nests rope_theta in rope_parameters (clockwork/engine/model.py:21-29)
        rope_params = raw.get("rope_parameters")
        if rope_params:
            rope_type = rope_params.get("rope_type", "default")
            if rope_type != "default":
                raise NotImplementedError(f"rope_type {rope_type!r} is not supported")
            theta = float(rope_params["rope_theta"])
        else:
            scaling = raw.get("rope_scaling")
            if scaling and scaling.get("rope_type", scaling.get("type", "default")) != "default":
                raise NotImplementedError(f"rope_scaling {scaling!r} is not supported")
            theta = _require(raw, "rope_theta", float)
        eos = raw.get("eos_token_id")  # clockwork/engine/llm_engine.py:24-32
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(
            vocab_size=_require(raw, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=_require(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=int(head_dim),
            intermediate_size=_require(raw, "intermediate_size", int),
            rms_norm_eps=_require(raw, "rms_norm_eps", float),
            rope_theta=theta,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            eos_token_ids=eos_ids,
            max_position_embeddings=raw.get("max_position_embeddings"),
        )

    def to_raw(self) -> dict[str, Any]:
        raw: dict[str, Any] = {
            "architectures": [Qwen2Architecture.name],
            "model_type": "qwen2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "use_sliding_window": False,
        }
        if self.max_position_embeddings is not None:
            raw["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            raw["eos_token_id"] = (
                self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
            )
        return raw


def _shape(**sizes) -> dict[str, Any]:
    return dict(sizes, architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_act="silu", use_sliding_window=False)


class Qwen2Architecture:
    name = "Qwen2ForCausalLM"

    # config.json contents of the sizes that the benchmarks and the command line know by name
    named_shapes = {
        "qwen2.5-1.5b": _shape(num_hidden_layers=28, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                               head_dim=128, intermediate_size=8960, vocab_size=151936, rope_theta=1000000.0,
                               rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=32768),
        "qwen2.5-7b": _shape(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
                             head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1000000.0,
                             rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=32768),
        "qwen2.5-32b": _shape(num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                              head_dim=128, intermediate_size=27648, vocab_size=152064, rope_theta=1000000.0,
                              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=32768),
        "tiny": _shape(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                       tie_word_embeddings=True, max_position_embeddings=256),
    }
    layer_count_key = "num_hidden_layers"  # the config.json key that a "fewer layers" option changes

    def parse_config(self, raw: dict[str, Any]) -> Qwen2Config:
        return Qwen2Config.from_raw(raw)

    def model_spec(self, config: Qwen2Config) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": config.hidden_size, "eps": config.rms_norm_eps})
        position = PartSpec(
            "rope_neox", {"theta": config.rope_theta, "rotary_dim": config.head_dim}
        )
        mixer = PartSpec(
            "attention",
            {
                "hidden_size": config.hidden_size,
                "num_heads": config.num_attention_heads,
                "num_kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim,
                "qkv_bias": True,  # clockwork/engine/model.py:74-76
                "o_bias": False,  # clockwork/engine/model.py:77
                "scale": config.head_dim**-0.5,  # clockwork/engine/model.py:73
                "window": None,  # full causal attention
                "position": position,
            },
        )
        ffn = PartSpec(
            "swiglu",
            {"hidden_size": config.hidden_size, "intermediate_size": config.intermediate_size},
        )
        layers = [
            LayerSpec(
                block="prenorm_residual",
                mixer=mixer,
                ffn=ffn,
                mixer_norm=norm,
                ffn_norm=norm,
                prefix=f"model.layers.{i}",
            )
            for i in range(config.num_hidden_layers)
        ]
        return ModelSpec(
            architecture=self.name,
            vocab_size=config.vocab_size,
            hidden_size=config.hidden_size,
            layers=layers,
            schedule=sequential_schedule(config.num_hidden_layers),
            final_norm=norm,
            tie_word_embeddings=config.tie_word_embeddings,
            eos_token_ids=config.eos_token_ids,
            max_position_embeddings=config.max_position_embeddings,
            raw=config.to_raw(),
        )


register_architecture(Qwen2Architecture(), replace=True)
