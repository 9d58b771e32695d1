"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it opens requests in the
cache manager, hands the step function what each line says, and closes requests when they end.
The reference has nothing equivalent; the closest are its test helpers
(``tests/test_hf_equivalence.py:26-43``).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: ``<out>/<step>.f32`` (little-endian float32 [wanted, vocab]) for steps that want
something, and a line ``done <step>`` on standard output after every step.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import Iterable, TextIO

import numpy as np
import torch

from ..cache.manager import CacheManager
from .loading import load_model
from .step import ModelRunner, StepEntry

MAX_LIVE_REQUESTS = 4


class TraceSession:
    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, page_size: int = 16,
                 device: str = "cuda:0", max_live: int = MAX_LIVE_REQUESTS) -> None:
        if max_tokens <= 0:
            raise ValueError("--max-tokens must be positive")
        self.model = load_model(model_dir, dtype, device)
        num_pages = (max_tokens + page_size - 1) // page_size
        self.cache = CacheManager(
            self.model.cache_needs(), num_pages=num_pages, page_size=page_size, dtype=self.model.dtype,
            device=device, num_state_slots=max_live, watermark=0.0,
        )
        self.runner = ModelRunner(self.model, self.cache)

    def run_step(self, record: dict) -> np.ndarray | None:
        entries = []
        for item in record.get("entries", []):
            rid = str(item["id"])
            if rid not in self.cache.requests:
                self.cache.open(rid)
            entries.append(StepEntry(rid, [int(t) for t in item["tokens"]], [int(w) for w in item.get("want", [])]))
        logits = self.runner.step(entries)
        out = None
        if logits is not None:
            out = logits.to("cpu", torch.float32).numpy()
        self.runner.check_status()
        for rid in record.get("end", []):
            self.cache.close(str(rid))
        return out


def replay(session: TraceSession, lines: Iterable[str], out_dir: str | Path, log: TextIO = sys.stdout) -> None:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = session.run_step(record)
        if logits is not None:
            logits.astype("<f4").tofile(out_dir / f"{step}.f32")
        print(f"done {step}", file=log, flush=True)


def main(argv: list[str] | None = None) -> int:
    import argparse

    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 1
    if 64 % args.page_size:
        print("trace_run: --page-size must divide 64", file=sys.stderr)
        return 1
    print("trace_run: loading model and kernels", file=sys.stderr, flush=True)
    session = TraceSession(args.model, args.dtype, args.max_tokens, args.page_size, args.device)
    print("trace_run: ready", file=sys.stderr, flush=True)
    replay(session, sys.stdin, args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
