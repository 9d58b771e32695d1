"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it opens requests in the
cache manager, hands the step function what each line says, and closes requests when they end.
Steps in which every request brings exactly one token go through the captured CUDA graphs that
generation uses for such steps (``--no-graphs``: through the uncaptured step function instead).
The reference has nothing equivalent; the closest are its test helpers
(``tests/test_hf_equivalence.py:26-43``).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: ``<out>/<step>.f32`` (little-endian float32 [wanted, vocab]) for steps that want
something, and a line ``done <step>`` on standard output after every step.

Two optional extensions exercise the cache manager's sharing of pages:

* ``"fork": [{"from": "a", "to": "b"}]`` in a record: before the step's entries run, request ``b``
  is created as a copy of ``a`` that shares all of ``a``'s pages; whoever writes into a shared page
  first gets a copy of it (``clockwork/kvcache/block_manager.py:56-83``).
* ``--prefix-cache``: whole pages of every request's tokens are recorded in the prefix cache after
  each step, and the tokens a request brings when it first appears are looked up there
  (``clockwork/radix/cache.py:36-70``): the whole pages that match (never all of the tokens) are
  taken over instead of being computed.  Logits wanted at taken-over places are not produced; the
  file ``<out>/<step>.cached.json`` then says how many tokens of which request were taken over.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import Iterable, TextIO

import numpy as np
import torch

from ..cache.allocator import OutOfPages
from ..cache.manager import CacheManager
from ..cache.prefix import PrefixCache
from .loading import load_model
from .step import ModelRunner, StepEntry

MAX_LIVE_REQUESTS = 4
BUDGET_GRANULE = 64  # --max-tokens counts each request rounded up to a multiple of this (or of the page size)


class TraceSession:
    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, page_size: int = 16,
                 device: str = "cuda:0", max_live: int = MAX_LIVE_REQUESTS, graphs: bool = True,
                 prefix_cache: bool = False) -> None:
        if max_tokens <= 0:
            raise ValueError("--max-tokens must be positive")
        if page_size <= 0:
            raise ValueError("--page-size must be positive")
        self.model = load_model(model_dir, dtype, device)
        num_pages = (max_tokens + page_size - 1) // page_size
        if BUDGET_GRANULE % page_size and page_size % BUDGET_GRANULE:
            # a request's last page may reach past its count rounded up to 64: one page more per live request
            num_pages += max_live
        self.cache = CacheManager(
            self.model.cache_needs(), num_pages=num_pages, page_size=page_size, dtype=self.model.dtype,
            device=device, num_state_slots=max_live, watermark=0.0,
        )
        self.runner = ModelRunner(self.model, self.cache)
        self.uses_graphs = graphs and self.runner.enable_graphs(max_ctx=num_pages * page_size, max_batch=max_live)
        self.prefix: PrefixCache | None = None
        if prefix_cache:
            if len(self.cache.groups) != 1 or self.cache.groups[0].need.window is not None or self.cache.state.needs:
                raise ValueError("--prefix-cache needs a model whose layers all keep every key (one group of pages)")
            self.prefix = PrefixCache(self.cache.groups[0].allocator, page_size)
        self._history: dict[str, list[int]] = {}  # tokens of each live request so far (prefix cache only)

    # ---- one record ---------------------------------------------------------------------------------
    def _open(self, rid: str, tokens: list[int]) -> int:
        """A request's first appearance.  Returns how many of ``tokens`` the prefix cache supplied."""
        if self.prefix is None:
            self.cache.open(rid)
            return 0
        match = self.prefix.match(tokens)
        self.cache.open(rid, shared_prefix=match.pages)
        self._history[rid] = list(tokens[: match.num_tokens])
        return match.num_tokens

    def _run(self, entries: list[StepEntry]) -> torch.Tensor | None:
        runner = self.runner
        wanted = sum(len(e.want) for e in entries)
        if (self.uses_graphs and runner.can_use_graph(entries)
                and all(self.cache.get(e.request_id).num_computed + 1 <= runner.graph_max_ctx for e in entries)):
            runner.decode_with_graph(entries, None)
            if not wanted:
                return None
            rows = [i for i, e in enumerate(entries) if e.want]
            return runner.last_graph.logits[rows]
        return runner.step(entries)

    def run_step(self, record: dict) -> tuple[np.ndarray | None, dict[str, int]]:
        for fork in record.get("fork", []):
            parent, child = str(fork["from"]), str(fork["to"])
            self.cache.fork(self.cache.get(parent), child)
            if self.prefix is not None:
                self._history[child] = list(self._history[parent])
        entries, cached = [], {}
        for item in record.get("entries", []):
            rid = str(item["id"])
            tokens = [int(t) for t in item["tokens"]]
            want = [int(w) for w in item.get("want", [])]
            if rid not in self.cache.requests:
                taken = self._open(rid, tokens)
                if taken:
                    cached[rid] = taken
                    tokens = tokens[taken:]
                    want = [w - taken for w in want if w >= taken]
            if self.prefix is not None:
                self._history[rid].extend(tokens)
            entries.append(StepEntry(rid, tokens, want))
        try:
            logits = self._run(entries)
        except OutOfPages:
            # pages that only the prefix cache still holds are not free: give the idle ones back and retry
            if self.prefix is None or self.prefix.evict(self.cache.num_pages) == 0:
                raise
            logits = self._run(entries)
        out = None
        if logits is not None:
            out = logits.to("cpu", torch.float32).numpy()
        self.runner.check_status()
        if self.prefix is not None:
            for e in entries:
                req = self.cache.get(e.request_id)
                self.prefix.insert(self._history[e.request_id][: req.num_computed], req.tables[0])
        for rid in record.get("end", []):
            shared = self.cache.close(str(rid))
            if self.prefix is not None:
                self.prefix.release(shared)
                self._history.pop(str(rid), None)
        return out, cached


def replay(session: TraceSession, lines: Iterable[str], out_dir: str | Path, log: TextIO = sys.stdout) -> None:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits, cached = session.run_step(record)
        if logits is not None:
            logits.astype("<f4").tofile(out_dir / f"{step}.f32")
        if cached:
            (out_dir / f"{step}.cached.json").write_text(json.dumps(cached))
        print(f"done {step}", file=log, flush=True)


def main(argv: list[str] | None = None) -> int:
    import argparse

    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64, or to the page size if larger)")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-live", type=int, default=MAX_LIVE_REQUESTS, help="most requests live at a time")
    parser.add_argument("--no-graphs", action="store_true",
                        help="run single-token steps through the uncaptured step function too")
    parser.add_argument("--prefix-cache", action="store_true",
                        help="share whole pages of equal leading tokens between requests (see the module text)")
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 1
    print("trace_run: loading model and kernels", file=sys.stderr, flush=True)
    try:
        session = TraceSession(args.model, args.dtype, args.max_tokens, args.page_size, args.device, args.max_live,
                               graphs=not args.no_graphs, prefix_cache=args.prefix_cache)
    except ValueError as exc:
        print(f"trace_run: {exc}", file=sys.stderr)
        return 1
    print("trace_run: ready", file=sys.stderr, flush=True)
    replay(session, sys.stdin, args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
