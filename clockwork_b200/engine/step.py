"""The step function: one flat batch of (request, its next tokens) through the model.

A step may hold portions of prompts beside single decoded tokens, cut anywhere.  It runs only
the tokens it is given; everything earlier comes from the cache.  It returns float32 logits at
the wanted places only.

The reference runs one forward per prefilling sequence and then one batched decode forward
(``clockwork/engine/model_runner.py:48-58``, ``68-132``), although its model accepts a mixed
batch (``clockwork/engine/model.py:103-118`` loops over per-sequence query lengths).  Here the
mixed batch is the only form: a decoded token is a portion of length one.  Inputs per step, as
in ``model_runner.py:72-91`` and ``98-124``: token ids, positions, slot mapping, block tables,
context lengths and the rows whose logits are wanted, uploaded in one copy from pinned memory.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops
from ..cache.manager import NO_PAGE, CacheManager
from ..ops.library import launch_count
from ..parts.base import StepContext
from ..parts.model import DecoderModel


@dataclass
class StepEntry:
    request_id: str
    tokens: list[int]  # the request's next tokens, in order
    want: list[int] = field(default_factory=list)  # places among ``tokens`` whose logits are wanted


def _pad4(n: int) -> int:
    return (n + 3) & ~3


@dataclass
class PreparedStep:
    ctx: StepContext
    token_ids: torch.Tensor  # int32 [N]
    logit_rows: torch.Tensor | None  # int32 [R]
    requests: list
    ctx_lens: list[int]


class StepBuilder:
    """Turns entries into the device-side description of a step (one upload from pinned memory)."""

    def __init__(self, cache: CacheManager, dtype: torch.dtype, device, status: torch.Tensor) -> None:
        self.cache = cache
        self.dtype = dtype
        self.device = torch.device(device)
        self.status = status
        self._pinned: torch.Tensor | None = None
        self._copy_done: torch.cuda.Event | None = None
        self.last_upload_bytes = 0

    def _staging(self, n_ints: int) -> torch.Tensor:
        if self._copy_done is not None:
            self._copy_done.synchronize()  # the last step's upload has left the staging buffer
        if self._pinned is None or self._pinned.numel() < n_ints:
            self._pinned = torch.empty(max(n_ints, 4096), dtype=torch.int32, pin_memory=True)
        return self._pinned

    def requests_of(self, entries: list[StepEntry]) -> list:
        """The entries' requests, with room reserved for the tokens they bring; refuses a request that
        appears twice and wanted places outside an entry's tokens."""
        cache = self.cache
        reqs = []
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            req = cache.get(e.request_id)
            cache.reserve(req, req.num_computed + len(e.tokens))
            reqs.append(req)
            bad = [w for w in e.want if not 0 <= w < len(e.tokens)]
            if bad:
                raise ValueError(f"request {e.request_id!r}: wanted places {bad} outside its {len(e.tokens)} tokens")
        return reqs

    def prepare(self, entries: list[StepEntry]) -> PreparedStep:
        cache = self.cache
        reqs = self.requests_of(entries)
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        N = sum(q_lens)
        starts = [r.num_computed for r in reqs]
        ctx_lens = [s + q for s, q in zip(starts, q_lens)]
        G = len(cache.groups)
        max_blocks = max(1, max((len(r.tables[g]) for r in reqs for g in range(G)), default=1))
        R = sum(len(e.want) for e in entries)

        # layout of the one staging buffer (every segment starts on a 16-byte boundary)
        seg = {}
        off = 0
        for name, size in (("tokens", N), ("positions", N), ("tok_seq", N), ("q_start", S + 1),
                           ("ctx_lens", S), ("rows", R), ("state", S)):
            seg[name] = (off, size)
            off += _pad4(size)
        for g in range(G):
            seg[f"slots{g}"] = (off, N)
            off += _pad4(N)
            seg[f"tables{g}"] = (off, S * max_blocks)
            off += _pad4(S * max_blocks)
        host = self._staging(off)
        h = host.numpy()

        def put(name, values):
            o, size = seg[name]
            h[o : o + size] = values

        put("tokens", np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=N))
        put("positions", np.concatenate([np.arange(s, s + q, dtype=np.int32) for s, q in zip(starts, q_lens)]))
        put("tok_seq", np.repeat(np.arange(S, dtype=np.int32), q_lens))
        q_start = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        put("q_start", q_start)
        put("ctx_lens", ctx_lens)
        put("rows", [int(q_start[i]) + w for i, e in enumerate(entries) for w in e.want])
        put("state", [r.state_slot if r.state_slot is not None else 0 for r in reqs])
        ps = cache.page_size
        for g in range(G):
            slots = np.empty(N, dtype=np.int32)
            tables = np.full((S, max_blocks), NO_PAGE, dtype=np.int32)
            for i, r in enumerate(reqs):
                table = np.asarray(r.tables[g], dtype=np.int32)
                tables[i, : len(table)] = table
                pos = np.arange(starts[i], ctx_lens[i], dtype=np.int32)
                pages = table[pos // ps]
                if (pages == NO_PAGE).any():
                    raise RuntimeError(f"request {r.request_id!r}: a token lands in a page that was given back")
                slots[q_start[i] : q_start[i + 1]] = pages * ps + pos % ps
            put(f"slots{g}", slots)
            put(f"tables{g}", tables.reshape(-1))

        dev = torch.empty(off, dtype=torch.int32, device=self.device)
        dev.copy_(host[:off], non_blocking=True)
        self.last_upload_bytes = off * 4
        if self._copy_done is None:
            self._copy_done = torch.cuda.Event()
        self._copy_done.record()

        def view(name):
            o, size = seg[name]
            return dev[o : o + size]

        ctx = StepContext(
            dtype=self.dtype, device=self.device, status=self.status, num_tokens=N, num_seqs=S,
            positions=view("positions"), tok_seq=view("tok_seq"), q_start=view("q_start"),
            ctx_lens=view("ctx_lens"), q_lens_host=q_lens, ctx_lens_host=ctx_lens,
            max_q_len=max(q_lens), max_ctx_len=max(ctx_lens),
        )
        state_slots = view("state").to(torch.int64) if cache.state.needs else None
        ctx.views = cache.views(
            [view(f"tables{g}").view(S, max_blocks) for g in range(G)],
            [view(f"slots{g}") for g in range(G)],
            state_slots, [r.state_slot for r in reqs] if cache.state.needs else [],
        )
        return PreparedStep(ctx, view("tokens"), view("rows") if R else None, reqs, ctx_lens)

    def commit(self, prepared: PreparedStep) -> None:
        """The step's tokens are in the cache now: advance the requests, let windows give pages back."""
        for r, end in zip(prepared.requests, prepared.ctx_lens):
            r.num_computed = end
            self.cache.release_behind_window(r, end)


def fresh_row(position: int, last_token: int, draws: int = 0, seed: int = 0, temperature: float = 0.0,
              top_k: int = 0, top_p: float = 1.0) -> tuple:
    """One request's column of the device state table, in the table's field order, as int32 words."""
    seed &= (1 << 64) - 1
    bits = np.array([temperature, top_p], dtype=np.float32).view(np.int32)
    lo, hi = seed & 0xFFFFFFFF, seed >> 32
    return (position, last_token, draws, lo - (1 << 32) if lo >= 1 << 31 else lo, hi - (1 << 32) if hi >= 1 << 31 else hi,
            int(bits[0]), max(0, int(top_k)), int(bits[1]))


class DecodeGraph:
    """One captured CUDA graph of a single-token step for a fixed number of rows: the step's inputs are
    derived on the device from the per-request state table (``csrc/request_state.cu``), then the
    model's forward pass, then sampling, which writes the new tokens back into the table.

    What the host supplies lives in the front part of one int32 buffer, uploaded in one copy and only
    when something in it changed: which state slot each row belongs to (< 0: padding), the block-table
    rows, the parts' per-step scalars, and for rows flagged ``fresh`` the column that overwrites the
    request's state first (after a prompt or a preemption, or when the caller supplies the token).  A
    step that only advances the same requests by one token needs no upload."""

    def __init__(self, runner: "ModelRunner", batch: int, max_ctx: int, greedy: bool) -> None:
        cache, model = runner.cache, runner.model
        self.batch, self.greedy = batch, greedy
        self.max_blocks = (max_ctx + cache.page_size - 1) // cache.page_size
        G = len(cache.groups)
        F = len(ops.REQUEST_STATE_FIELDS)
        # values that the parts' kernels read from device memory and that change with the live requests
        # (``Part.step_scalars``): one word each
        self._scalar_rules = model.step_scalars()
        uploaded = [("row_slot", batch), ("fresh", batch), ("fresh_values", F * batch),
                    *((f"scalar:{name}", 1) for name in self._scalar_rules),
                    *((f"tables{g}", batch * self.max_blocks) for g in range(G))]
        derived = [("tokens", batch), ("positions", batch), ("tok_seq", batch), ("ctx_lens", batch), ("temperature", batch),
                   ("top_k", batch), ("top_p", batch), ("uniform", batch), *((f"slots{g}", batch) for g in range(G)),
                   ("q_start", batch + 1), ("rows", batch)]
        seg, off = {}, 0
        for name, size in uploaded:
            seg[name] = (off, size)
            off += _pad4(size)
        self.upload_words = off
        for name, size in derived:
            seg[name] = (off, size)
            off += _pad4(size)
        self.seg, self.size = seg, off
        self.host = torch.zeros(self.upload_words, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(off, dtype=torch.int32, device=runner.device)
        h = self.host.numpy()
        self.h = {name: h[o : o + n] for name, (o, n) in seg.items() if o < self.upload_words}
        self.h["fresh_values"] = self.h["fresh_values"].reshape(F, batch)
        for g in range(G):
            self.h[f"tables{g}"] = self.h[f"tables{g}"].reshape(batch, self.max_blocks)
            self.h[f"tables{g}"][:] = NO_PAGE
        self.h["row_slot"][:] = -1
        self.upload_bytes = self.upload_words * 4
        self.uploads = 0  # how many replays needed an upload
        self._uploaded = torch.cuda.Event()
        self._dirty = True
        self._filled = 0
        # which request's table each row holds and how much of it, so that a step writes only the
        # pages a request gained since its last step
        self._row_owner: list[list] = [[None] * batch for _ in range(G)]  # per group and row: (request, table length held, its table_epoch)

        def view(name):
            o, n = seg[name]
            return self.dev[o : o + n]

        view("q_start").copy_(torch.arange(batch + 1, dtype=torch.int32))
        view("rows").copy_(torch.arange(batch, dtype=torch.int32))
        ctx = StepContext(
            dtype=model.dtype, device=runner.device, status=runner.status, num_tokens=batch, num_seqs=batch,
            positions=view("positions"), tok_seq=view("tok_seq"), q_start=view("q_start"), ctx_lens=view("ctx_lens"),
            q_lens_host=[1] * batch, ctx_lens_host=[max_ctx] * batch, max_q_len=1, max_ctx_len=max_ctx,
            inputs_from_device=True,
        )
        tables = [view(f"tables{g}").view(batch, self.max_blocks) for g in range(G)]
        kv_slots = [view(f"slots{g}") for g in range(G)]
        # mixers with state of their own: row r's state is in slot row_slot[r] (padding rows use the scratch row)
        state_rows = torch.zeros(batch, dtype=torch.int64, device=runner.device) if cache.state.needs else None
        ctx.views = cache.views(tables, kv_slots, state_rows, [])
        for name, rule in self._scalar_rules.items():
            ctx.extras[name] = view(f"scalar:{name}")
            self.h[f"scalar:{name}"][0] = rule(batch, max_ctx)
        state = cache.state.request
        as_float = lambda name: view(name).view(torch.float32)  # noqa: E731

        def run():
            if state_rows is not None:
                row_slot = view("row_slot")
                state_rows.copy_(torch.where(row_slot < 0, cache.state.scratch_slot, row_slot))
            ops.step_from_state(view("row_slot"), view("fresh"), view("fresh_values").view(F, batch), state, tables, kv_slots,
                                cache.page_size, cache.num_pages, view("tokens"), view("positions"), view("ctx_lens"),
                                view("tok_seq"), as_float("temperature"), view("top_k"), as_float("top_p"),
                                as_float("uniform"), runner.status)
            # the logits of every row stay readable after a replay (trace replay reads them; generation
            # reads the sampled tokens only)
            logits = self.logits = model.forward(ctx, view("tokens"), view("rows"))
            into_state = (view("row_slot"), state)
            if greedy:
                return ops.argmax(logits, into_state=into_state)
            return ops.sample(logits, as_float("temperature"), view("top_k"), as_float("top_p"), as_float("uniform"),
                              into_state=into_state)

        self.dev[: self.upload_words].copy_(self.host)  # all rows padding: the warm-up and the capture touch no request
        before = launch_count()
        run()  # eager warm-up: scratch buffers and kernel attributes are set up outside the capture
        self.kernels = launch_count() - before
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = run()
        torch.cuda.synchronize()

    def fill(self, cache: CacheManager, reqs, fresh_rows: list[tuple] | None) -> None:
        """What the host supplies for a step of these requests, one row each, written into the pinned
        buffer (it depends on the requests' positions and pages only, so it can be done while the step
        before is still running).  ``fresh_rows``: per row the column that replaces the request's device
        state first (``fresh_row``), or None when every row just goes on from the step before."""
        n = self._filled = len(reqs)
        self._uploaded.synchronize()  # the last upload has left the pinned buffer
        h, ps = self.h, cache.page_size
        dirty = False
        slots = np.fromiter((r.state_slot for r in reqs), dtype=np.int32, count=n)
        if (h["row_slot"][:n] != slots).any() or (h["row_slot"][n:] != -1).any():
            # (state is kept by slot, not by row: requests may change rows, or graphs, and go on)
            h["row_slot"][:n] = slots
            h["row_slot"][n:] = -1
            dirty = True
        if h["fresh"].any():
            h["fresh"][:] = 0  # (cleared on the device by the step that used them)
        if fresh_rows is not None:
            h["fresh"][:n] = 1
            h["fresh_values"][:, :n] = np.array(fresh_rows, dtype=np.int64).T.astype(np.int32)
            dirty = True
        pos = np.fromiter((r.num_computed for r in reqs), dtype=np.int32, count=n)
        rows = np.arange(n)
        for g in range(len(cache.groups)):
            tables = h[f"tables{g}"]
            owners = self._row_owner[g]
            for i, r in enumerate(reqs):
                # a row is rewritten only from where the request's table grew since the row last held it
                # (most steps: nowhere)
                table = r.tables[g]
                held = min(len(table), self.max_blocks)  # (pages beyond the graph's context bound are not this step's)
                owner = owners[i]
                if owner is not None and owner[0] is r and owner[1] == held and owner[2] == r.table_epoch:
                    continue
                same = owner is not None and owner[0] is r and owner[2] == r.table_epoch and owner[1] <= held
                have = owner[1] if same else 0
                tables[i, have:held] = table[have:held]
                owners[i] = (r, held, r.table_epoch)
                dirty = True
            pages = tables[rows, pos // ps]
            if (pages == NO_PAGE).any():
                bad = reqs[int(np.argmax(pages == NO_PAGE))]
                raise RuntimeError(f"request {bad.request_id!r}: a token lands in a page that was given back")
        longest = int(pos.max()) + 1
        for name, rule in self._scalar_rules.items():
            value = rule(n, longest)
            if h[f"scalar:{name}"][0] != value:
                h[f"scalar:{name}"][0] = value
                dirty = True
        self._dirty = self._dirty or dirty

    def launch(self) -> torch.Tensor:
        """The upload, if the host's part changed, and the replay.  Returns the sampled tokens of the live rows."""
        if self._dirty:
            self.dev[: self.upload_words].copy_(self.host, non_blocking=True)
            self._uploaded.record()
            self._dirty = False
            self.uploads += 1
            self.last_upload_bytes = self.upload_bytes
        else:
            self.last_upload_bytes = 0
        self.graph.replay()
        return self.out[: self._filled]


class PortionGraph:
    """One captured CUDA graph of a step that holds prompt portions: up to ``tokens`` tokens of up to
    ``seqs`` requests with contexts up to ``max_ctx``, logits at up to ``rows`` places.  Such a step's
    kernels are many and small when the portions are short (a prompt of a few hundred tokens, a portion
    beside decoded tokens), and launching them one by one from the host takes longer than they run.

    Everything the step's kernels need to know about its contents lives in one int32 device buffer,
    written on the host and uploaded in one copy before every replay: the arrays of an uncaptured step
    (``StepBuilder.prepare``) at fixed lengths, the parts' per-step scalars and the parts' per-step
    arrays (``Part.step_arrays``).  Unused token rows carry token 0 at position 0 with no cache slot,
    belong to no request, and are computed and ignored; unused requests have no tokens.  ``singles``:
    whether the steps that replay this graph hold requests that bring one token (parts may serve those
    apart from the portions, as attention does with its decode kernel)."""

    def __init__(self, runner: "ModelRunner", tokens: int, seqs: int, rows: int, max_ctx: int, singles: bool) -> None:
        cache, model = runner.cache, runner.model
        self.tokens, self.seqs, self.rows, self.max_ctx, self.singles = tokens, seqs, rows, max_ctx, singles
        self.max_blocks = (max_ctx + cache.page_size - 1) // cache.page_size
        G = len(cache.groups)
        self._scalar_rules = model.step_scalars()
        # (with single tokens in the step, at most PORTION_MAX_PORTIONS requests bring more: see _portion_graph_key)
        self._arrays = model.step_arrays(tokens, seqs, cache.page_size, runner.PORTION_MAX_PORTIONS if singles else None, max_ctx)
        layout = [("tokens", tokens), ("positions", tokens), ("tok_seq", tokens), ("q_start", seqs + 1), ("ctx_lens", seqs),
                  ("rows", rows), ("state", seqs), *((f"scalar:{name}", 1) for name in self._scalar_rules),
                  *((("array", key), words) for key, (words, _, _) in self._arrays.items())]
        for g in range(G):
            layout += [(f"slots{g}", tokens), (f"tables{g}", seqs * self.max_blocks)]
        seg, off = {}, 0
        for name, size in layout:
            seg[name] = (off, size)
            off += _pad4(size)
        self.seg, self.size = seg, off
        self.host = torch.zeros(off, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(off, dtype=torch.int32, device=runner.device)
        h = self.host.numpy()
        self.h = {name: h[o : o + n] for name, (o, n) in seg.items()}
        for g in range(G):
            self.h[f"tables{g}"] = self.h[f"tables{g}"].reshape(seqs, self.max_blocks)
        self.upload_bytes = off * 4
        self._uploaded = torch.cuda.Event()
        self._filled_rows = 0

        def view(name):
            o, n = seg[name]
            return self.dev[o : o + n]

        ctx = StepContext(
            dtype=model.dtype, device=runner.device, status=runner.status, num_tokens=tokens, num_seqs=seqs,
            positions=view("positions"), tok_seq=view("tok_seq"), q_start=view("q_start"), ctx_lens=view("ctx_lens"),
            q_lens_host=[], ctx_lens_host=[], max_q_len=tokens, max_ctx_len=max_ctx,
        )
        ctx.extras["captured_portions"] = {"singles": singles}
        for name in self._scalar_rules:
            ctx.extras[name] = view(f"scalar:{name}")
        for key, (_, _, present) in self._arrays.items():
            ctx.extras[key] = present(view(("array", key)))
        tables = [view(f"tables{g}").view(seqs, self.max_blocks) for g in range(G)]
        kv_slots = [view(f"slots{g}") for g in range(G)]
        state_rows = torch.zeros(seqs, dtype=torch.int64, device=runner.device) if cache.state.needs else None
        ctx.views = cache.views(tables, kv_slots, state_rows, [])

        def run():
            if state_rows is not None:
                state_rows.copy_(view("state"))
            return model.forward(ctx, view("tokens"), view("rows"))

        self._write_padding(cache, 0, 0, 0)
        self.dev.copy_(self.host)  # no request at all: the warm-up and the capture touch no cache slot
        before = launch_count()
        run()  # eager warm-up: scratch buffers and kernel attributes are set up outside the capture
        self.kernels = launch_count() - before
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = run()
        torch.cuda.synchronize()

    def _write_padding(self, cache: CacheManager, n: int, s: int, r: int) -> None:
        """Everything behind the first ``n`` tokens, ``s`` requests and ``r`` wanted rows."""
        h = self.h
        h["tokens"][n:] = 0
        h["positions"][n:] = 0
        h["tok_seq"][n:] = -1
        h["q_start"][s + 1 :] = n
        h["ctx_lens"][s:] = 0
        h["rows"][r:] = 0
        h["state"][s:] = cache.state.scratch_slot
        for g in range(len(cache.groups)):
            h[f"slots{g}"][n:] = -1
            h[f"tables{g}"][s:] = NO_PAGE
        if n == 0:  # (the capture: no request, no work)
            h["q_start"][:] = 0
            for name in self._scalar_rules:
                h[f"scalar:{name}"][0] = self._scalar_rules[name](1, 1)
            for key, (_, fill, _) in self._arrays.items():
                h[("array", key)][:] = fill([], [])

    def fill(self, cache: CacheManager, entries: list[StepEntry], reqs: list) -> list[int]:
        """The step's description written into the pinned buffer.  Returns the context lengths after the step."""
        self._uploaded.synchronize()  # the last upload has left the pinned buffer
        h, ps = self.h, cache.page_size
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        N = sum(q_lens)
        starts = [r.num_computed for r in reqs]
        ctx_lens = [a + q for a, q in zip(starts, q_lens)]
        rows = [w for e in entries for w in e.want]
        R = len(rows)
        h["tokens"][:N] = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=N)
        h["positions"][:N] = np.concatenate([np.arange(a, a + q, dtype=np.int32) for a, q in zip(starts, q_lens)])
        h["tok_seq"][:N] = np.repeat(np.arange(S, dtype=np.int32), q_lens)
        q_start = np.zeros(S + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        h["q_start"][: S + 1] = q_start
        h["ctx_lens"][:S] = ctx_lens
        h["rows"][:R] = [int(q_start[i]) + w for i, e in enumerate(entries) for w in e.want]
        h["state"][:S] = [r.state_slot if r.state_slot is not None else cache.state.scratch_slot for r in reqs]
        for g in range(len(cache.groups)):
            slots, tables = h[f"slots{g}"], h[f"tables{g}"]
            tables[:S] = NO_PAGE
            for i, r in enumerate(reqs):
                table = np.asarray(r.tables[g], dtype=np.int32)
                # (a request may hold pages for tokens far beyond this step's: the scheduler reserves a
                # whole prompt's at admission; the step reads the table up to its context bound only)
                held = min(len(table), self.max_blocks)
                tables[i, :held] = table[:held]
                pos = np.arange(starts[i], ctx_lens[i], dtype=np.int32)
                pages = table[pos // ps]
                if (pages == NO_PAGE).any():
                    raise RuntimeError(f"request {r.request_id!r}: a token lands in a page that was given back")
                slots[q_start[i] : q_start[i + 1]] = pages * ps + pos % ps
        self._write_padding(cache, N, S, R)
        single_ctx = [c for q, c in zip(q_lens, ctx_lens) if q == 1]
        for name, rule in self._scalar_rules.items():
            # (the scalars speak of the requests that bring one token: the decode kernel's share of the step)
            h[f"scalar:{name}"][0] = rule(max(1, len(single_ctx)), max(single_ctx, default=1))
        for key, (_, fill, _) in self._arrays.items():
            h[("array", key)][:] = fill(q_lens, ctx_lens)
        self._filled_rows = R
        return ctx_lens

    def launch(self) -> torch.Tensor | None:
        """The upload and the replay.  Returns the logits of the wanted rows (a view of the graph's own
        output buffer: the next replay of the same graph overwrites it), or None when none is wanted."""
        self.dev.copy_(self.host, non_blocking=True)
        self._uploaded.record()
        self.graph.replay()
        return self.logits[: self._filled_rows] if self._filled_rows else None


class ModelRunner:
    """The step function over a model and a cache manager."""

    def __init__(self, model: DecoderModel, cache: CacheManager) -> None:
        if model.device.type != "cuda":
            raise RuntimeError("the step function runs on a CUDA device only (there is no CPU path)")
        ops.library()  # fail now, loudly, if the kernels cannot be built or loaded
        self.model = model
        self.cache = cache
        self.device = model.device
        self.status = cache.status if cache.status is not None else ops.device_status(self.device)
        self.builder = StepBuilder(cache, model.dtype, self.device, self.status)
        self.steps_run = 0
        self.graphs: dict[tuple[int, bool, int], DecodeGraph] = {}  # (batch bucket, greedy, context tier)
        self.graph_max_ctx = 0  # set by enable_graphs
        self.portions_captured = False  # whether short steps with prompt portions replay captured graphs too
        self.graph_max_batch = 0
        self.graph_kernel_launches = 0  # kernels replayed through graphs (for accounting)
        self.last_graph: DecodeGraph | None = None  # the graph of the last captured step that ran
        self.portion_graphs: dict[tuple, PortionGraph] = {}  # (tokens, requests, rows, context tier, singles apart)
        self.portion_graph_steps = 0  # steps with prompt portions that replayed a captured graph
        self.last_upload_bytes = 0
        self.uploaded_bytes = 0  # host-to-device bytes of all steps so far

    def enable_graphs(self, max_ctx: int, max_batch: int) -> bool:
        """Let steps in which every request brings exactly one token replay a captured CUDA graph
        (one per batch-size bucket).  Only for models whose parts are all safe to capture (a mixer with
        state of its own is, if it finds its rows through the device-side slot list of its view)."""
        if not self.model.graph_safe():
            return False
        self.graph_max_ctx, self.graph_max_batch = max_ctx, max_batch
        self.model.reserve_for_steps(max_batch, max_ctx)  # scratch that captured graphs point at is set up once
        self.portions_captured = self.model.dtype == torch.bfloat16 and self.model.graph_safe_portions()
        return True

    def can_use_graph(self, entries: list[StepEntry]) -> bool:
        return (self.graph_max_batch > 0 and 0 < len(entries) <= self.graph_max_batch
                and all(len(e.tokens) == 1 for e in entries))

    def decode_with_graph(self, entries: list[StepEntry], sampling_rows: list[tuple] | None = None) -> torch.Tensor:
        """One single-token step for every entry through the captured graph, sampling included, the
        tokens given by the caller.  ``sampling_rows``: per entry (temperature, top_k, top_p, seed, draws),
        or None for greedy.  Returns the sampled tokens (device int32 [len(entries)])."""
        cache = self.cache
        fresh = []
        for i, e in enumerate(entries):
            position = cache.get(e.request_id).num_computed
            if sampling_rows is None:
                fresh.append(fresh_row(position, e.tokens[0]))
            else:
                temperature, top_k, top_p, seed, draws = sampling_rows[i]
                fresh.append(fresh_row(position, e.tokens[0], draws, seed, temperature, top_k, top_p))
        return self.launch_decode(self.prepare_decode([e.request_id for e in entries], fresh, greedy=sampling_rows is None))

    def prepare_decode(self, request_ids: list[str], fresh_rows: list[tuple] | None, greedy: bool = True):
        """The first half of a captured step: slots reserved, graph chosen, the host's part of its inputs
        written.  It needs the requests' positions only, so the engine may call it for step N+1 while
        step N runs (after step N's launch: positions are advanced at launch).  ``fresh_rows``: see
        ``DecodeGraph.fill``."""
        cache = self.cache
        reqs = []
        for rid in request_ids:
            req = cache.get(rid)
            cache.reserve(req, req.num_computed + 1)
            if req.num_computed + 1 > self.graph_max_ctx:
                raise ValueError(f"request {rid!r} outgrew the context the decode graphs were captured for")
            reqs.append(req)
        n = len(reqs)
        bucket = 1
        while bucket < n:
            bucket *= 2
        bucket = min(bucket, max(self.graph_max_batch, n))
        # Graphs are captured per context tier (a power of two, at least 1024): the tier bounds the
        # attention grid and the block-table width, and lets short contexts run the attention variant
        # whose CTAs are small enough to start beside the preceding product's.  A request that grows
        # past its tier moves the step to the next tier's graph (captured on first use).
        longest = max(r.num_computed + 1 for r in reqs)
        tier = 1024
        while tier < longest:
            tier *= 2
        tier = min(tier, self.graph_max_ctx)
        key = (bucket, greedy, tier)
        graph = self.graphs.get(key)
        if graph is None:
            graph = self.graphs[key] = DecodeGraph(self, bucket, tier, greedy=greedy)
        graph.fill(cache, reqs, fresh_rows)
        return graph, reqs

    def launch_decode(self, prepared) -> torch.Tensor:
        """The second half: the upload (if the host's part of the inputs changed), the replay; positions
        advance.  Returns the sampled tokens on the device (the graph's own output buffer: the next
        replay of the same graph overwrites it)."""
        graph, reqs = prepared
        cache = self.cache
        out = graph.launch()
        self.last_graph = graph
        self.graph_kernel_launches += graph.kernels
        self.last_upload_bytes = graph.last_upload_bytes
        self.uploaded_bytes += graph.last_upload_bytes
        for r in reqs:
            r.num_computed += 1
            cache.release_behind_window(r, r.num_computed)
        self.steps_run += 1
        return out

    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Run the entries as one batch.  Returns float32 logits [wanted rows, vocab] in the order
        of the entries and of each entry's ``want``, or None when nothing is wanted."""
        entries = [e for e in entries if e.tokens]
        if not entries:
            return None
        graph_key = self._portion_graph_key(entries)
        if graph_key is not None:
            return self._step_with_portion_graph(entries, graph_key)
        prepared = self.builder.prepare(entries)
        logits = self.model.forward(prepared.ctx, prepared.token_ids, prepared.logit_rows)
        self.builder.commit(prepared)
        self.last_upload_bytes = self.builder.last_upload_bytes
        self.uploaded_bytes += self.builder.last_upload_bytes
        self.steps_run += 1
        return logits

    # A step with prompt portions replays a captured graph: always when it is short enough to be bound by
    # the host's launches (up to PORTION_TOKEN_BUCKETS[-1] tokens, padded to the next bucket), and up to
    # PORTION_MAX_TOKENS when a multiple of PORTION_LONG_STEP tokens is at most PORTION_LONG_WASTE above its
    # size (the gaps between launches cost a long step about 5 %; more padding than that would cost more).
    # The small buckets are those of the products' token tiles: a prompt of 8 to 64 tokens, or the rest of one
    # behind a prefix-cache hit, costs 1.4 to 1.8 ms at the 1.5B sizes instead of the 2.2 ms of 128 tokens.
    PORTION_TOKEN_BUCKETS = (16, 32, 64, 128, 192, 256, 384, 512, 768, 1024)
    PORTION_MAX_TOKENS = 4096
    PORTION_LONG_STEP = 256
    PORTION_LONG_WASTE = 0.04
    PORTION_SEQ_BUCKETS = (8, 64)
    PORTION_MAX_LOGITS = 1 << 28  # float32 logits that a captured step may keep (1 GiB)
    PORTION_MAX_GRAPHS = 32       # captured steps kept at a time
    PORTION_MAX_PORTIONS = 8      # requests with more than one token in a captured step that also holds single tokens

    def _portion_token_bucket(self, tokens: int) -> int | None:
        if tokens <= self.PORTION_TOKEN_BUCKETS[-1]:
            return next(b for b in self.PORTION_TOKEN_BUCKETS if b >= tokens)
        bucket = -(-tokens // self.PORTION_LONG_STEP) * self.PORTION_LONG_STEP
        if bucket <= self.PORTION_MAX_TOKENS and bucket <= tokens * (1 + self.PORTION_LONG_WASTE):
            return bucket
        return None

    def _portion_graph_key(self, entries: list[StepEntry]) -> tuple | None:
        if not self.portions_captured or len(entries) > self.PORTION_SEQ_BUCKETS[-1]:
            return None
        tokens = sum(len(e.tokens) for e in entries)
        bucket = self._portion_token_bucket(tokens)
        if bucket is None or tokens == len(entries):  # (all single tokens: the decode graphs' steps)
            return None
        longest = max(self.cache.get(e.request_id).num_computed + len(e.tokens) for e in entries)
        if longest > self.graph_max_ctx:
            return None
        seqs = next(b for b in self.PORTION_SEQ_BUCKETS if b >= len(entries))
        wanted = sum(len(e.want) for e in entries)
        rows = seqs if wanted <= seqs else max(seqs, bucket)  # one row per request, or any rows
        if rows * self.model.spec.vocab_size > self.PORTION_MAX_LOGITS:
            return None  # (logits at many places of a long step: the graph would hold gigabytes for them)
        tier = 1024
        while tier < longest:
            tier *= 2
        tier = min(tier, self.graph_max_ctx)
        singles = any(len(e.tokens) == 1 for e in entries)
        if singles and sum(1 for e in entries if len(e.tokens) > 1) > self.PORTION_MAX_PORTIONS:
            return None  # (a captured step with single tokens has work lists for this many portions)
        return bucket, seqs, rows, tier, singles

    def capture_ahead(self, decode_batches=(), prompt_tokens=(), max_ctx: int = 1024, greedy: bool = True) -> int:
        """Captures, before any request needs them, the graphs of single-token steps of these batch sizes
        and of one-prompt steps of these token counts, for contexts up to ``max_ctx`` (a graph is otherwise
        captured at its first use, a few tenths of a second that this one step pays for).  Touches no
        request and no cache slot.  Returns the number of graphs captured."""
        if not self.graph_max_batch:
            return 0
        tier = 1024
        while tier < max_ctx:
            tier *= 2
        tier = min(tier, self.graph_max_ctx)
        made = 0
        for n in decode_batches:
            bucket = 1
            while bucket < n:
                bucket *= 2
            key = (min(bucket, max(self.graph_max_batch, n)), greedy, tier)
            if key not in self.graphs:
                self.graphs[key] = DecodeGraph(self, key[0], tier, greedy=greedy)
                made += 1
        for tokens in prompt_tokens:
            bucket = self._portion_token_bucket(tokens) if self.portions_captured else None
            if bucket is None:
                continue
            key = (bucket, self.PORTION_SEQ_BUCKETS[0], self.PORTION_SEQ_BUCKETS[0], tier, False)
            if key not in self.portion_graphs and len(self.portion_graphs) < self.PORTION_MAX_GRAPHS:
                self.portion_graphs[key] = PortionGraph(self, *key)
                made += 1
        return made

    def _step_with_portion_graph(self, entries: list[StepEntry], key: tuple) -> torch.Tensor | None:
        reqs = self.builder.requests_of(entries)
        graph = self.portion_graphs.pop(key, None)
        if graph is None:
            # every captured step keeps its own activations: the least recently used ones make room
            while len(self.portion_graphs) >= self.PORTION_MAX_GRAPHS:
                del self.portion_graphs[next(iter(self.portion_graphs))]
            graph = PortionGraph(self, *key)
        self.portion_graphs[key] = graph  # (the dictionary's order is the order of last use)
        ctx_lens = graph.fill(self.cache, entries, reqs)
        logits = graph.launch()
        self.builder.commit(PreparedStep(None, None, None, reqs, ctx_lens))
        self.graph_kernel_launches += graph.kernels
        self.portion_graph_steps += 1
        self.last_upload_bytes = graph.upload_bytes
        self.uploaded_bytes += graph.upload_bytes
        self.steps_run += 1
        return logits

    def check_status(self) -> None:
        """Raise if any kernel of a step reported since the last check: an index out of range (which
        it skipped) or a device-side wait that gave up.  The step's kernels, the tensor-core products
        included, all report into the device's one status word (``ops.device_status``)."""
        ops.raise_on_status(self.status)
