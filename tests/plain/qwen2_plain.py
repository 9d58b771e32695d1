"""A plain, slow Qwen2 forward pass: whole sequences, no cache, one function per part, float32
(or float64) torch on the CPU.  It is the yardstick of the tests and shares no code with
``clockwork_b200``: it reads the model folder with its own few lines and computes every part
from the reference's formulas, each cited below by the reference's file:line.

It was compared once with the reference's own ``clockwork.engine.model.Qwen2ForCausalLM`` on
tiny random models; the outputs of that run are in ``tests/golden`` together with the script
that made them, and ``tests/test_plain_vs_golden.py`` re-checks them.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32}


def read_model_dir(model_dir, dtype=torch.float32):
    """(config dict, {name: tensor as ``dtype``}) from config.json + model.safetensors."""
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    blob = (model_dir / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + n])
    header.pop("__metadata__", None)
    tensors = {}
    for name, info in header.items():
        b, e = info["data_offsets"]
        raw = bytearray(blob[8 + n + b : 8 + n + e])
        t = torch.frombuffer(raw, dtype=_ST_DTYPES[info["dtype"]]).reshape(info["shape"])
        tensors[name] = t.to(dtype) if t.is_floating_point() else t
    return config, tensors


def head_dim_of(config) -> int:
    # clockwork/engine/model.py:17-18
    return config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]


def rms_norm(x, weight, eps):
    # clockwork/engine/model.py:44-49
    variance = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_cos_sin(positions, head_dim, theta, dtype):
    # clockwork/engine/model.py:171-175 (inv_freq, float32) and :186-191 (angles, cos, sin)
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x):
    # clockwork/engine/model.py:32-35
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x, cos, sin):
    # clockwork/engine/model.py:92-95; x [T, heads, hd], cos/sin [T, hd]
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def causal_attention(q, k, v, scale, window=None, q_offset=None):
    """q [Tq, nh, hd], k/v [Tk, nkv, hd] -> [Tq, nh, hd].
    clockwork/kernels/attention.py:45-65: GQA by repeat_interleave (:35-42), scores scaled after
    the dot product (:56), query row i at absolute position Tk - Tq + i sees keys j <= that
    (:57-63), softmax, P.V (:64-65).  ``window`` (not in the reference, which has full attention
    only) additionally hides keys more than window-1 positions back."""
    tq, nh, _ = q.shape
    tk, nkv, _ = k.shape
    rep = nh // nkv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k) * scale
    offset = tk - tq if q_offset is None else q_offset
    q_pos = torch.arange(tq)[:, None] + offset
    k_pos = torch.arange(tk)[None, :]
    hidden = k_pos > q_pos
    if window is not None:
        hidden = hidden | (k_pos <= q_pos - window)
    scores = scores.masked_fill(hidden, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", probs, v)


def exact(x):
    return x


def to_bfloat16_and_back(x):
    """Rounds activations the way a bfloat16 run stores them between kernels.  Passing this as
    ``rnd`` makes the plain implementation show how much bfloat16 storage alone moves the logits of
    a given model, which is the yardstick for the bfloat16 engine's tolerance in the tests."""
    return x.to(torch.bfloat16).to(torch.float32)


def attention_block(x, w, prefix, config, positions, window=None, rnd=exact):
    # clockwork/engine/model.py:79-128 with kv_cache=None
    nh, nkv, hd = config["num_attention_heads"], config["num_key_value_heads"], head_dim_of(config)
    t = x.shape[0]
    q = rnd(x @ w[f"{prefix}.q_proj.weight"].T + w[f"{prefix}.q_proj.bias"]).view(t, nh, hd)
    k = rnd(x @ w[f"{prefix}.k_proj.weight"].T + w[f"{prefix}.k_proj.bias"]).view(t, nkv, hd)
    v = rnd(x @ w[f"{prefix}.v_proj.weight"].T + w[f"{prefix}.v_proj.bias"]).view(t, nkv, hd)
    cos, sin = rope_cos_sin(positions, hd, float(config["rope_theta"]), x.dtype)
    q, k = rnd(apply_rope(q, cos, sin)), rnd(apply_rope(k, cos, sin))
    out = rnd(causal_attention(q, k, v, hd**-0.5, window=window))
    return out.reshape(t, nh * hd) @ w[f"{prefix}.o_proj.weight"].T


def swiglu_mlp(x, w, prefix, rnd=exact):
    # clockwork/engine/model.py:62-63
    gate = x @ w[f"{prefix}.gate_proj.weight"].T
    up = x @ w[f"{prefix}.up_proj.weight"].T
    return rnd(torch.nn.functional.silu(gate) * up) @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(h, w, i, config, positions, rnd=exact):
    # clockwork/engine/model.py:147-154
    p = f"model.layers.{i}"
    eps = config["rms_norm_eps"]
    h = h + attention_block(rnd(rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)), w, f"{p}.self_attn", config,
                            positions, rnd=rnd)
    h = h + swiglu_mlp(rnd(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps)), w, f"{p}.mlp", rnd=rnd)
    return h


def final_hidden_states(config, w, token_ids, rnd=exact):
    """[T, hidden] after the last layer and the final norm (clockwork/engine/model.py:193-204)."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    h = w["model.embed_tokens.weight"][ids]
    for i in range(config["num_hidden_layers"]):
        h = decoder_layer(h, w, i, config, positions, rnd=rnd)
    return rnd(rms_norm(h, w["model.norm.weight"], config["rms_norm_eps"]))


def output_head(config, w):
    # clockwork/engine/model.py:216-218: the head is the embedding matrix when the model ties them
    return w["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else w["lm_head.weight"]


def logits_at(config, w, token_ids, rows, rnd=exact):
    """[len(rows), vocab] logits of one whole sequence at the given positions only
    (clockwork/engine/model.py:229-233 applies the head to the selected rows)."""
    h = final_hidden_states(config, w, token_ids, rnd=rnd)
    return h[torch.as_tensor(rows, dtype=torch.long)] @ output_head(config, w).T


def all_position_logits(config, w, token_ids, rnd=exact):
    """[T, vocab] logits of one whole sequence (clockwork/engine/model.py:193-204, 220-233)."""
    return final_hidden_states(config, w, token_ids, rnd=rnd) @ output_head(config, w).T


def greedy_generate(config, w, prompt, num_new):
    # clockwork/engine/model_runner.py:136-137 (first maximal index), recomputing the whole
    # sequence every step as tests/test_hf_equivalence.py:58-69 does
    ids = list(prompt)
    for _ in range(num_new):
        ids.append(int(all_position_logits(config, w, ids)[-1].argmax()))
    return ids[len(prompt):]


def sampling_probs(logits, temperature, top_k=-1, top_p=1.0):
    # clockwork/engine/model_runner.py:147-164
    logits = logits.to(torch.float32) / temperature
    if 0 < top_k < logits.shape[-1]:
        kth = torch.topk(logits, top_k).values[-1]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        sorted_logits, sorted_indices = torch.sort(logits, descending=True)
        cumulative = torch.softmax(sorted_logits, dim=-1).cumsum(dim=-1)
        sorted_removed = cumulative > top_p
        sorted_removed[1:] = sorted_removed[:-1].clone()
        sorted_removed[0] = False
        removed = torch.zeros_like(sorted_removed)
        removed[sorted_indices] = sorted_removed
        logits = logits.masked_fill(removed, float("-inf"))
    return torch.softmax(logits, dim=-1)


def sample_with_uniform(logits, temperature, top_k, top_p, u):
    """The token whose cumulative probability (in index order) first exceeds ``u``: the
    inverse-CDF draw that stands for the reference's ``torch.multinomial``
    (clockwork/engine/model_runner.py:145)."""
    if temperature == 0.0:
        return int(logits.argmax())
    probs = sampling_probs(logits, temperature, top_k, top_p).double()
    cdf = probs.cumsum(0)
    idx = int((cdf > u * float(cdf[-1])).nonzero()[0])
    return idx
