"""One layer at the sizes of the two wider models that the benchmark description names (Qwen2.5-7B: hidden
3584, 28 query and 4 KV heads of 128, feed-forward 18944; Qwen2.5-32B: hidden 5120, 40 query and 8 KV heads,
feed-forward 27648, eps 1e-5; both with an output head of its own) against the plain implementation, in
bfloat16 (the float32 run's kernels take their sizes as loop bounds and are held at every other size by the
other tests; a float64 reference at these widths would take minutes).  Every size of the layer is the real one; the vocabulary is cut to 8,003 entries (no
kernel but the two that read the tables depends on it, and they are held at 151,936 elsewhere) so that the
model folder stays small.  The kernels meet other sizes here than at the 1.5B layer: products with inner
dimensions of 3584, 5120, 18944 and 27648 (other splits over thread-block clusters, other tile counts per
CTA pair, other numbers of slabs that the norm adds up), q/k/v rows of 4608 and 7168, decode attention
with seven and five query heads per KV head.

Random weights with the q and k projections scaled up, as in ``tests/test_real_sizes_gpu.py``.
"""

import json

import pytest
import torch

from tests.test_real_sizes_gpu import SHARPEN, SparseTrace, compare, plain_references, some_places, tokens
from tests.trace_tools import cut, round_up, run_trace

pytestmark = pytest.mark.gpu

VOCAB = 8003
PAGE = 16


def one_layer_config(shape: str) -> dict:
    from clockwork_b200 import models  # noqa: F401  (registers the architecture and its named sizes)
    from clockwork_b200.config.registry import shape_config

    raw = shape_config(shape, 1)
    raw["vocab_size"] = VOCAB
    return raw


def write_model(folder, config: dict, seed: int):
    """config.json + model.safetensors with random bfloat16 weights drawn by torch (half a billion values: its
    generator is several times faster than the one behind the package's random-weights mode)."""
    from clockwork_b200.config.registry import spec_from_raw
    from clockwork_b200.parts.model import tensor_decls_for_spec
    from clockwork_b200.weights import save_safetensors

    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for decl in tensor_decls_for_spec(spec_from_raw(config)):
        if decl.optional:
            continue
        assert decl.init in ("norm", "linear", "bias", "embedding"), decl
        t = torch.randn(decl.shape, generator=g)
        t = 1.0 + 0.1 * t if decl.init == "norm" else 0.02 * t
        if ".q_proj." in decl.name or ".k_proj." in decl.name:
            t = t * SHARPEN
        tensors[decl.name] = t.to(torch.bfloat16)
    (folder / "config.json").write_text(json.dumps(config))
    save_safetensors(folder / "model.safetensors", tensors)
    return folder


@pytest.fixture(scope="module", params=["qwen2.5-7b", "qwen2.5-32b"])
def wide(request, tmp_path_factory):
    folder = write_model(tmp_path_factory.mktemp(request.param.replace(".", "_")), one_layer_config(request.param), seed=23)
    return request.param, folder, plain_references(folder)


@pytest.mark.parametrize("dtype", ["bfloat16"])
def test_one_layer_of_the_wider_models(dtype, wide, tmp_path):
    """A prompt whole; a prompt and then 24 single tokens (the captured single-token steps); a prompt in
    portions of changing size (129 to 257 tokens among them, which take the products whose splits the next
    norm adds up, and two tokens); and three requests mixed, portions beside single tokens."""
    shape, folder, references = wide
    seqs = {"whole": tokens(200, 1, VOCAB), "tail": tokens(150, 2, VOCAB), "cuts": tokens(470, 3, VOCAB)}
    tr = SparseTrace()
    tr.sparse_step([("whole", seqs["whole"], some_places(200) + [63, 64, 127, 128])], end=["whole"])
    tr.sparse_step([("tail", seqs["tail"][:126], [0, 125])])
    for i, t in enumerate(seqs["tail"][126:]):
        tr.sparse_step([("tail", [t], [0])], end=["tail"] if 126 + i == 149 else [])
    portions = cut(seqs["cuts"], [130, 2, 257, 17, 64])
    for i, portion in enumerate(portions):
        tr.sparse_step([("cuts", portion, some_places(len(portion)))], end=["cuts"] if i == len(portions) - 1 else [])
    mixed = {"m0": tokens(150, 10, VOCAB), "m1": tokens(90, 11, VOCAB), "m2": tokens(140, 12, VOCAB)}
    tr.sparse_step([("m0", mixed["m0"][:100], [0, 99])])
    tr.sparse_step([("m0", mixed["m0"][100:101], [0]), ("m1", mixed["m1"][:70], [69])])
    tr.sparse_step([("m0", mixed["m0"][101:102], [0]), ("m1", mixed["m1"][70:71], [0]), ("m2", mixed["m2"][:129], [0, 128])])
    for i in range(10):
        step = [("m0", mixed["m0"][102 + i : 103 + i], [0]), ("m1", mixed["m1"][71 + i : 72 + i], [0]),
                ("m2", mixed["m2"][129 + i : 130 + i], [0])]
        tr.sparse_step(step, end=list(mixed) if i == 9 else [])
    used = {"m0": mixed["m0"][:112], "m1": mixed["m1"][:81], "m2": mixed["m2"][:139]}
    seqs.update(used)
    budget = max(round_up(470, 64), sum(round_up(len(t), 64) for t in used.values()))
    out = run_trace(folder, dtype, budget, tr.steps, tmp_path / "out", VOCAB, PAGE, timeout=900)
    compare(tr, out, seqs, references, dtype, f"one layer of {shape}")
