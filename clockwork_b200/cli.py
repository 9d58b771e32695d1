"""Command line.

    python -m clockwork_b200 generate --config configs/qwen2.5-1.5b.yaml --set num_blocks=1024 \\
        --prompt-ids 1,2,3 --prompt-ids 4,5 --max-tokens 16 --temperature 0.8 --seed 1
    python -m clockwork_b200 generate --model DIR --prompt-len 32 --num-prompts 4
    python -m clockwork_b200 random-model --shape qwen2.5-1.5b --seed 0 --out DIR
    python -m clockwork_b200 replay --model DIR --dtype float32 --out DIR --max-tokens 256 < trace.jsonl

``--config`` (a YAML profile with model/cache/scheduler sections) and ``--set KEY=VALUE`` (override
any model, cache or scheduler field) have the names and meanings of the reference's launcher
(``scripts/serve.py:33-49``); its ``--host``/``--port`` belong to the HTTP server, which this engine
does not have.  Sampling options are the fields of ``SamplingParams``.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

def shape_names() -> list[str]:
    from . import models  # noqa: F401  (registers architectures)
    from .config.registry import named_shapes

    return sorted(named_shapes())


def shape_config(name: str, num_layers: int | None = None) -> dict:
    """config.json of a size that a registered architecture knows by name."""
    from . import models  # noqa: F401
    from .config import registry

    try:
        return registry.shape_config(name, num_layers)
    except ValueError as exc:
        raise SystemExit(str(exc)) from None


def _engine_config(args):
    from .config import EngineConfig

    if args.config:
        cfg = EngineConfig.from_yaml(args.config)
        if args.model:
            cfg.model.model = args.model
    elif args.model:
        cfg = EngineConfig.defaults(args.model)
    else:
        raise SystemExit("give --config or --model")
    try:
        cfg.apply_pairs(args.overrides)
    except ValueError as exc:
        raise SystemExit(str(exc)) from None
    return cfg


def _cmd_generate(args) -> int:
    from .engine import LLMEngine
    from .sampling import SamplingParams

    cfg = _engine_config(args)
    engine = LLMEngine(cfg)
    vocab = engine.model.spec.vocab_size
    prompts: list[list[int]] = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    if args.prompt_len:
        import random

        rng = random.Random(args.seed if args.seed is not None else cfg.model.seed)
        prompts += [[rng.randrange(vocab) for _ in range(args.prompt_len)] for _ in range(args.num_prompts)]
    if not prompts:
        raise SystemExit("no prompts: give --prompt-ids or --prompt-len")
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                            top_k=args.top_k, stop_token_ids=args.stop_token_ids, ignore_eos=args.ignore_eos,
                            seed=args.seed)
    for out in engine.generate(prompts, params):
        print(json.dumps({"request_id": out.request_id, "prompt_token_ids": out.prompt_token_ids,
                          "token_ids": out.token_ids, "finish_reason": out.finish_reason,
                          "num_cached_tokens": out.num_cached_tokens}))
    if args.stats:
        print(json.dumps(engine.stats()), file=sys.stderr)
    return 0


def _cmd_random_model(args) -> int:
    from .weights import write_random_model

    raw = json.loads(Path(args.config_json).read_text()) if args.config_json else shape_config(args.shape, args.num_layers)
    out = write_random_model(args.out, raw, seed=args.seed, store_dtype=args.store_dtype)
    print(out)
    return 0


def _cmd_replay(args) -> int:
    from .engine.trace import main as trace_main

    return trace_main(["--model", args.model, "--dtype", args.dtype, "--out", args.out,
                       "--max-tokens", str(args.max_tokens), "--page-size", str(args.page_size)])


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="clockwork_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    g.add_argument("--config", help="YAML profile (model/cache/scheduler sections)")
    g.add_argument("--model", help="model folder (overrides the profile's model.model)")
    g.add_argument("--set", dest="overrides", action="append", default=[], metavar="KEY=VALUE",
                   help="override any model, cache, or scheduler field, e.g. --set num_blocks=1024")
    g.add_argument("--prompt-ids", action="append", default=[], metavar="ID,ID,...")
    g.add_argument("--prompt-len", type=int, default=0, help="add --num-prompts random prompts of this length")
    g.add_argument("--num-prompts", type=int, default=1)
    g.add_argument("--max-tokens", type=int, default=64)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--stop-token-ids", type=lambda s: [int(t) for t in s.split(",") if t], default=[])
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--stats", action="store_true", help="print engine counters to stderr at the end")
    g.set_defaults(fn=_cmd_generate)

    r = sub.add_parser("random-model", help="write config.json + model.safetensors with random weights")
    r.add_argument("--shape", default="tiny", help=f"one of {shape_names()}")
    r.add_argument("--config-json", help="a config.json to use instead of --shape")
    r.add_argument("--num-layers", type=int, default=None)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--out", required=True)
    r.set_defaults(fn=_cmd_random_model)

    t = sub.add_parser("replay", help="trace replay (same as bin/trace_run)")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--page-size", type=int, default=16)
    t.set_defaults(fn=_cmd_replay)

    args = parser.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
