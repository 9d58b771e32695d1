"""Drives ``bin/trace_run`` the way a user does: one process, a JSON line per step on its standard
input, waiting for ``done <step>`` before the next line, logits read back from ``<out>/<step>.f32``."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
TRACE_RUN = ROOT / "bin" / "trace_run"


def round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class TraceOutputs(dict):
    """{step: float32 [rows, vocab]} plus ``cached``: {step: {request: tokens the prefix cache supplied}}."""

    def __init__(self) -> None:
        super().__init__()
        self.cached: dict[int, dict[str, int]] = {}


def run_trace(model_dir, dtype: str, max_tokens: int, steps: list[dict], out_dir, vocab: int,
              page_size: int | None = None, timeout: float = 600.0, extra_args: tuple[str, ...] = ()) -> TraceOutputs:
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(max_tokens), *extra_args]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        for record in steps:
            proc.stdin.write(json.dumps(record) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            if line != f"done {record['step']}":
                proc.stdin.close()
                err = proc.stderr.read()
                raise AssertionError(f"trace_run answered {line!r} to step {record['step']}\n{err[-3000:]}")
        proc.stdin.close()
        rc = proc.wait(timeout=timeout)
        err = proc.stderr.read()
        assert rc == 0, f"trace_run exited with {rc}\n{err[-3000:]}"
    finally:
        if proc.poll() is None:
            proc.kill()
    out = TraceOutputs()
    for record in steps:
        number = record["step"]
        sidecar = out_dir / f"{number}.cached.json"
        cached = json.loads(sidecar.read_text()) if sidecar.exists() else {}
        if cached:
            out.cached[number] = cached
        # logits wanted at places that the prefix cache supplied are not produced
        wanted = sum(sum(1 for w in e.get("want", []) if w >= cached.get(e["id"], 0)) for e in record["entries"])
        path = out_dir / f"{number}.f32"
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == wanted * vocab, f"step {number}: {data.size} floats for {wanted} rows"
            out[number] = data.reshape(wanted, vocab)
        else:
            assert not path.exists(), f"step {number} wanted nothing but wrote a file"
    return out


class TraceBuilder:
    """Collects steps and remembers which request positions each step's wanted rows stand for."""

    def __init__(self) -> None:
        self.steps: list[dict] = []
        self._cursor: dict[str, int] = {}
        self._starts: list[dict[str, int]] = []  # per step: position of each entry's first token

    def step(self, portions: list[tuple[str, list[int], bool]], end: list[str] = (), fork: list[tuple[str, str]] = ()) -> None:
        """portions: (request id, its next tokens, want logits at every one of them?).
        fork: (parent, child) pairs; the child starts where the parent stands."""
        number = len(self.steps)
        for parent, child in fork:
            self._cursor[child] = self._cursor.get(parent, 0)
        entries, starts = [], {}
        for rid, tokens, want_all in portions:
            starts[rid] = self._cursor.get(rid, 0)
            self._cursor[rid] = starts[rid] + len(tokens)
            entries.append({"id": rid, "tokens": tokens, "want": list(range(len(tokens))) if want_all else []})
        record = {"step": number, "entries": entries, "end": list(end)}
        if fork:
            record["fork"] = [{"from": parent, "to": child} for parent, child in fork]
        self.steps.append(record)
        self._starts.append(starts)

    def gather(self, outputs: dict[int, np.ndarray], rid: str, length: int, first: int = 0) -> torch.Tensor:
        """The logits of positions [first, length) of a request, in order."""
        where: dict[int, tuple[int, int]] = {}
        cached_by_step = getattr(outputs, "cached", {})
        for record, starts in zip(self.steps, self._starts):
            cached = cached_by_step.get(record["step"], {})
            row = 0
            for e in record["entries"]:
                for w in e["want"]:
                    if w < cached.get(e["id"], 0):
                        continue
                    if e["id"] == rid:
                        where[starts[rid] + w] = (record["step"], row)
                    row += 1
        rows = []
        for pos in range(first, length):
            step, row = where[pos]
            rows.append(outputs[step][row])
        return torch.from_numpy(np.stack(rows))


def cut(tokens: list[int], sizes: list[int]) -> list[list[int]]:
    """Cuts tokens into portions of the given sizes, cycling through ``sizes``."""
    out, pos, i = [], 0, 0
    while pos < len(tokens):
        n = min(sizes[i % len(sizes)], len(tokens) - pos)
        out.append(tokens[pos : pos + n])
        pos += n
        i += 1
    return out
