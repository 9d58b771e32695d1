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


def run_trace(model_dir, dtype: str, max_tokens: int, steps: list[dict], out_dir, vocab: int,
              page_size: int | None = None, timeout: float = 600.0) -> dict[int, np.ndarray]:
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(max_tokens)]
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
    out = {}
    for record in steps:
        wanted = sum(len(e.get("want", [])) for e in record["entries"])
        path = out_dir / f"{record['step']}.f32"
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == wanted * vocab, f"step {record['step']}: {data.size} floats for {wanted} rows"
            out[record["step"]] = data.reshape(wanted, vocab)
        else:
            assert not path.exists(), f"step {record['step']} wanted nothing but wrote a file"
    return out


class TraceBuilder:
    """Collects steps and remembers which output row belongs to which (request, position)."""

    def __init__(self) -> None:
        self.steps: list[dict] = []
        self.where: dict[tuple[str, int], tuple[int, int]] = {}  # (request, position) -> (step, row)
        self._cursor: dict[str, int] = {}

    def step(self, portions: list[tuple[str, list[int], bool]], end: list[str] = ()) -> None:
        """portions: (request id, its next tokens, want logits at every one of them?)."""
        number = len(self.steps)
        entries, row = [], 0
        for rid, tokens, want_all in portions:
            start = self._cursor.get(rid, 0)
            want = list(range(len(tokens))) if want_all else []
            for w in want:
                self.where[(rid, start + w)] = (number, row)
                row += 1
            self._cursor[rid] = start + len(tokens)
            entries.append({"id": rid, "tokens": tokens, "want": want})
        self.steps.append({"step": number, "entries": entries, "end": list(end)})

    def gather(self, outputs: dict[int, np.ndarray], rid: str, length: int) -> torch.Tensor:
        rows = []
        for pos in range(length):
            step, row = self.where[(rid, pos)]
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
