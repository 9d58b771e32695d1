"""The two tiny Qwen2 configurations of the tests.  They differ in every size and option:
layer count, width, head counts and group size, head size (B's is not hidden/heads), feed-forward
width (B's is no multiple of 16), vocabulary, rope base, norm eps, tied/untied head, page size."""

from __future__ import annotations

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256,
    "hidden_act": "silu", "use_sliding_window": False,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 200, "vocab_size": 320, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 512,
    "hidden_act": "silu", "use_sliding_window": False,
}
TINY = {"A": (TINY_A, 0, 4), "B": (TINY_B, 1, 8)}  # name -> (config.json, weight seed, page size)


def tokens_for(name: str, length: int, salt: int = 0) -> list[int]:
    """Deterministic pseudo-random token ids (a small LCG; no library generator involved)."""
    vocab = TINY[name][0]["vocab_size"]
    state = (hash_name(name) + 7919 * salt + 104729 * length) & 0x7FFFFFFF
    out = []
    for _ in range(length):
        state = (1103515245 * state + 12345) & 0x7FFFFFFF
        out.append((state >> 8) % vocab)
    return out


def hash_name(name: str) -> int:
    return sum((i + 1) * ord(c) for i, c in enumerate(name)) * 2654435761 & 0x7FFFFFFF


def reference_checkout():
    """Folder of a checkout of the reference project, for the tests that compare with its own code:
    the environment variable CLOCKWORK_REFERENCE, else a folder ``reference`` beside this repository."""
    import os
    from pathlib import Path

    named = os.environ.get("CLOCKWORK_REFERENCE")
    return Path(named) if named else Path(__file__).resolve().parents[2] / "reference"
