"""What ``bench.py`` promises on its command line and in its record, as far as that can be held without a GPU:
more than one GPU is refused with one line and exit code 2, options that belong to one part are refused
elsewhere, the ``config`` of the record is flat with at most 20 keys and names every size, and the
FLOP count of a prompt is the sum that it says it is."""

import importlib.util
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=300)


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_more_than_one_gpu_is_refused_with_one_line():
    done = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert done.returncode == 2
    assert len(done.stdout.strip().splitlines()) == 1 and "one GPU" in done.stdout


def test_options_of_one_part_are_refused_elsewhere():
    for args in (("--prompt-len", "4096"), ("--temperature", "0.8"), ("--only", "prefill", "--top-k", "5")):
        done = run(*args)
        assert done.returncode == 2 and "--only" in done.stdout, (args, done.stdout, done.stderr[-500:])


def test_the_record_s_config_is_flat_and_names_every_size():
    bench = load_bench()
    from clockwork_b200 import models  # noqa: F401  (registers the architecture and its named sizes)
    from clockwork_b200.config.registry import shape_config

    shape = shape_config("qwen2.5-1.5b")
    config = bench.config_record(shape, shape["num_hidden_layers"], 8, 1100, "measured")
    assert len(config) <= 20
    assert all(isinstance(v, (int, float, str, bool)) for v in config.values())
    sizes = {"layers": "num_hidden_layers", "hidden": "hidden_size", "heads": "num_attention_heads", "kv_heads": "num_key_value_heads",
             "head_dim": "head_dim", "intermediate": "intermediate_size", "vocab": "vocab_size"}
    for key, name in sizes.items():
        assert config[key] == shape[name]
    assert config["layers_full"] == 28 and config["global_batch"] == 8 and config["seq_len"] == 1280


def test_the_flops_of_a_prompt():
    bench = load_bench()
    shape = {"hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
             "num_hidden_layers": 3, "vocab_size": 1000}
    tokens = 10
    per_token_layer = 2 * (64 * (4 + 2 * 2) * 16 + 4 * 16 * 64 + 3 * 64 * 128)   # q/k/v, output, gate + up + down
    causal_pairs = tokens * (tokens + 1) // 2                                     # (query, key) pairs under the diagonal
    attention = 3 * causal_pairs * 4 * 16 * 2 * 2                                 # per pair and head: hd MACs for the score, hd for the value
    head = 2 * 64 * 1000                                                          # logits of the last token only
    assert bench.prefill_flops(shape, tokens) == 3 * tokens * per_token_layer + attention + head
