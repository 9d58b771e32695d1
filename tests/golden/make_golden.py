"""Makes tests/golden/*.npz: outputs of the reference's own model code on the tiny models.

    python tests/golden/make_golden.py /path/to/clockwork-checkout

It imports ``clockwork.engine.model.Qwen2ForCausalLM`` from the given checkout (torch on the
CPU, float32; a ``types.SimpleNamespace`` stands for the Hugging Face config object, so no
other package's model code is involved), loads the tiny random models that
``clockwork_b200.weights.write_random_model`` writes for the configurations of
``tests/tiny_configs.py``, and stores for each: the token ids, the reference's logits at every
position ([T, vocab] float32), its greedy continuation, and a checksum of the weights.
``tests/test_plain_vs_golden.py`` compares the plain implementation with these files.
"""

from __future__ import annotations

import sys
import tempfile
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from clockwork_b200.weights import write_random_model  # noqa: E402
from tests.plain.qwen2_plain import read_model_dir  # noqa: E402
from tests.tiny_configs import TINY, tokens_for  # noqa: E402

LENGTHS = {"A": 17, "B": 40}
GREEDY_PROMPT, GREEDY_NEW = 9, 12


def weight_checksum(weights) -> float:
    return float(sum(w.double().abs().sum() for _, w in sorted(weights.items())))


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from clockwork.engine.attn_metadata import AttentionMetadata
    from clockwork.engine.model import Qwen2ForCausalLM

    for name, (raw, seed, _page) in TINY.items():
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(tmp, raw, seed=seed)
            config, weights = read_model_dir(tmp)
        model = Qwen2ForCausalLM(SimpleNamespace(**config))
        missing, unexpected = model.load_state_dict(weights, strict=False)
        assert not unexpected and set(missing) <= {"lm_head.weight"}, (missing, unexpected)
        model.eval()
        tokens = tokens_for(name, LENGTHS[name])
        n = len(tokens)
        meta = AttentionMetadata(
            is_prefill=True, slot_mapping=torch.empty(0, dtype=torch.int64), block_tables=None,
            ctx_lens=None, query_lens=[n], seq_block_tables=[[]], logits_indices=torch.arange(n),
        )
        with torch.inference_mode():
            logits = model(torch.tensor(tokens), torch.arange(n), None, meta)
            ids = tokens[:GREEDY_PROMPT]
            for _ in range(GREEDY_NEW):
                last = model(torch.tensor(ids), torch.arange(len(ids)), None, None)
                ids.append(int(last[-1].argmax()))
        out = Path(__file__).parent / f"tiny_{name.lower()}.npz"
        np.savez_compressed(
            out, tokens=np.array(tokens, dtype=np.int32), logits=logits.numpy().astype(np.float32),
            greedy=np.array(ids[GREEDY_PROMPT:], dtype=np.int32), checksum=np.float64(weight_checksum(weights)),
        )
        print(f"wrote {out} ({out.stat().st_size} bytes)")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <folder of a checkout of the reference project>")
    main(sys.argv[1])
