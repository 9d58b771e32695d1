"""Generality of the parts, second helping: a feed-forward with routing (top-1 of three small experts,
router logits in float32) and a position encoding that is not the model's own (rotary with
interpolated positions), both defined in this file only, registered, written as a random model
folder, loaded and stepped whole, in portions and through the engine, without a change to the
framework's files.  A toy, not any real model."""

import pytest
import torch

from clockwork_b200 import EngineConfig, ops
from clockwork_b200.cache import CacheManager
from clockwork_b200.config import LayerSpec, ModelSpec, PartSpec, register_architecture, sequential_schedule
from clockwork_b200.engine import LLMEngine, ModelRunner, StepEntry, load_model
from clockwork_b200.parts import FeedForward, PositionEncoding, register_ffn, register_position
from clockwork_b200.sampling import SamplingParams
from clockwork_b200.weights import TensorDecl, write_random_model
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
EXPERTS = 3


class Top1RoutedFFN(FeedForward):
    """out[t] = p_e * down_e(silu(gate_e x_t) * up_e x_t) with e = argmax of the float32 router logits
    router_scale * x_t W_r^T and p_e its softmax probability.  Returns its contribution; the next norm adds it."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.h, self.i, self.router_scale = spec["hidden_size"], spec["intermediate_size"], spec["router_scale"]

    def tensor_decls(self):
        yield TensorDecl(self.name("router.weight"), (EXPERTS, self.h), "state32", "linear")  # kept in float32
        for e in range(EXPERTS):
            yield TensorDecl(self.name(f"experts.{e}.gate.weight"), (self.i, self.h), "matrix", "linear")
            yield TensorDecl(self.name(f"experts.{e}.up.weight"), (self.i, self.h), "matrix", "linear")
            yield TensorDecl(self.name(f"experts.{e}.down.weight"), (self.h, self.i), "matrix", "linear")

    def load_weights(self, fetch):
        self.router = fetch(self.name("router.weight"))
        self.experts = [tuple(fetch(self.name(f"experts.{e}.{p}.weight")) for p in ("gate", "up", "down"))
                        for e in range(EXPERTS)]

    def forward(self, ctx, x, stream):
        probs = torch.softmax(self.router_scale * (x.float() @ self.router.float().T), dim=-1)
        p, choice = probs.max(dim=-1)
        out = torch.zeros(x.shape[0], self.h, dtype=torch.float32, device=x.device)
        for e, (gate, up, down) in enumerate(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                xe = x[rows].float()
                act = torch.nn.functional.silu(xe @ gate.float().T) * (xe @ up.float().T)
                out[rows] = p[rows, None] * (act.to(x.dtype).float() @ down.float().T)
        return out.to(self.dtype)


class InterpolatedRotary(PositionEncoding):
    """Rotate-half rotary on positions divided by ``factor`` (position interpolation): the kernels take
    any float32 frequencies, so this encoding only has to hand over its own."""

    graph_safe = True

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.rotary_dim, theta, factor = int(spec["rotary_dim"]), float(spec["theta"]), float(spec["factor"])
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (theta**exponents) / factor).to(device)

    def apply_and_store(self, ctx, qkv, view, num_heads, num_kv_heads, head_dim):
        write = view is not None and view.write
        ops.rope_store(qkv, ctx.positions, view.slots if write else None, self.inv_freq, view.k_cache if write else None,
                       view.v_cache if write else None, num_heads, num_kv_heads, head_dim, self.rotary_dim, ctx.status,
                       write_cache=write)

    def fused_decode_args(self, head_dim):  # lets the decode attention kernel rotate by itself
        return (self.inv_freq, self.rotary_dim)


class ToyArchitecture:
    name = "ToyRoutedLM"

    def parse_config(self, raw):
        return raw

    def model_spec(self, raw):
        h = raw["hidden_size"]
        norm = PartSpec("rmsnorm", {"size": h, "eps": raw["eps"]})

        def attention(position):
            return PartSpec("attention", dict(hidden_size=h, num_heads=6, num_kv_heads=3, head_dim=16, qkv_bias=True,
                                              o_bias=False, position=position))

        layers = [
            LayerSpec("prenorm_residual", attention(PartSpec("toy_interpolated_rotary", dict(rotary_dim=16, theta=50.0, factor=4.0))),
                      PartSpec("toy_top1_routed", dict(hidden_size=h, intermediate_size=raw["ffn"], router_scale=raw["router_scale"])), norm, norm, "model.layers.0"),
            LayerSpec("prenorm_residual", attention(PartSpec("none", {})),
                      PartSpec("swiglu", dict(hidden_size=h, intermediate_size=raw["ffn"])), norm, norm, "model.layers.1"),
        ]
        return ModelSpec(self.name, raw["vocab_size"], h, layers, sequential_schedule(2), norm, tie_word_embeddings=False, raw=raw)


RAW = dict(architectures=["ToyRoutedLM"], hidden_size=40, vocab_size=70, eps=1e-6, ffn=56, router_scale=60.0)


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    register_ffn("toy_top1_routed", Top1RoutedFFN, replace=True)
    register_position("toy_interpolated_rotary", InterpolatedRotary, replace=True)
    register_architecture(ToyArchitecture(), replace=True)
    return write_random_model(tmp_path_factory.mktemp("toy_routed"), RAW, seed=11)


def plain_logits(folder, tokens):
    """Whole sequence, no cache; returns the logits and each token's router margin (top-1 minus top-2)."""
    _, w = plain.read_model_dir(folder)
    t, eps = len(tokens), RAW["eps"]
    positions = torch.arange(t)

    def attention(x, prefix, rotary):
        def proj(name, heads):
            return (x @ w[f"{prefix}.{name}.weight"].T + w[f"{prefix}.{name}.bias"]).view(t, heads, 16)

        q, k, v = proj("q_proj", 6), proj("k_proj", 3), proj("v_proj", 3)
        if rotary:
            cos, sin = plain.rope_cos_sin(positions.float() / 4.0, 16, 50.0, torch.float32)
            q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        return plain.causal_attention(q, k, v, 16**-0.5).reshape(t, 96) @ w[f"{prefix}.o_proj.weight"].T

    margins = []

    def routed(x, prefix):
        probs = torch.softmax(RAW["router_scale"] * (x @ w[f"{prefix}.router.weight"].T), dim=-1)
        top = probs.topk(2, dim=-1).values
        margins.append(top[:, 0] - top[:, 1])
        p, choice = probs.max(dim=-1)
        rows = []
        for i in range(t):
            e = int(choice[i])
            act = torch.nn.functional.silu(x[i] @ w[f"{prefix}.experts.{e}.gate.weight"].T) * (x[i] @ w[f"{prefix}.experts.{e}.up.weight"].T)
            rows.append(p[i] * (act @ w[f"{prefix}.experts.{e}.down.weight"].T))
        return torch.stack(rows)

    h = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    for i, (rotary, ffn) in enumerate([(True, routed), (False, lambda x, p: plain.swiglu_mlp(x, w, p))]):
        p = f"model.layers.{i}"
        h = h + attention(plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], eps), f"{p}.self_attn", rotary)
        h = h + ffn(plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), f"{p}.mlp")
    return plain.rms_norm(h, w["model.norm.weight"], eps) @ w["lm_head.weight"].T, margins[0]


def tokens(n, salt):
    return [(salt * 17 + i * i * 5 + 3 * i) % RAW["vocab_size"] for i in range(n)]


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-5), ("bfloat16", 5e-2)])
def test_toy_routed_model_steps_like_its_plain_form(toy_dir, dtype, tol):
    model = load_model(toy_dir, dtype)
    cache = CacheManager(model.cache_needs(), num_pages=32, page_size=4, dtype=model.dtype, device=DEV, num_state_slots=2)
    runner = ModelRunner(model, cache)
    a, b = tokens(41, 1), tokens(18, 2)
    (want_a, margin_a), (want_b, margin_b) = plain_logits(toy_dir, a), plain_logits(toy_dir, b)

    def safe_rows(margin):
        """Rows to compare: all in float32; in bfloat16 those before the first token whose routing is
        too close to call (its choice, and every later row through attention, may differ)."""
        if dtype == "float32":
            return len(margin)
        close = (margin < 0.05).nonzero().flatten()
        return int(close[0]) if close.numel() else len(margin)

    def run(plan):
        got, pos, data = {"a": [], "b": []}, {"a": 0, "b": 0}, {"a": a, "b": b}
        for step in plan:
            entries = []
            for rid, n in step.items():
                if rid not in cache.requests:
                    cache.open(rid)
                entries.append(StepEntry(rid, data[rid][pos[rid] : pos[rid] + n], list(range(n))))
                pos[rid] += n
            logits = runner.step(entries).cpu()
            runner.check_status()
            row = 0
            for rid, n in step.items():
                got[rid].append(logits[row : row + n])
                row += n
        for rid in list(cache.requests):
            cache.close(rid)
        cache.check_invariants()
        return {rid: torch.cat(rows) for rid, rows in got.items()}

    na, nb = safe_rows(margin_a), safe_rows(margin_b)
    assert na >= 8 and nb >= 8  # the comparison must not be empty
    for plan in ([{"a": 41}, {"b": 18}], [{"a": 7}, {"a": 2, "b": 9}, {"b": 1}, {"a": 30, "b": 1}, {"a": 1, "b": 7}, {"a": 1}]):
        got = run(plan)
        torch.testing.assert_close(got["a"][:na], want_a[:na], rtol=tol, atol=tol)
        torch.testing.assert_close(got["b"][:nb], want_b[:nb], rtol=tol, atol=tol)
    assert cache.num_free_pages() == [32]


def test_toy_routed_model_generates_through_the_engine(toy_dir):
    cfg = EngineConfig.defaults(str(toy_dir), dtype="float32", block_size=4, num_blocks=48, max_num_seqs=3,
                                max_num_batched_tokens=16, max_model_len=128)
    eng = LLMEngine(cfg)
    prompts = [tokens(13, 3), tokens(5, 4), tokens(21, 5)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for _ in range(6):
            ids.append(int(plain_logits(toy_dir, ids)[0][-1].argmax()))
        assert out.token_ids == ids[len(prompt):]
