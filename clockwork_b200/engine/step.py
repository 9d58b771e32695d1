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

    def prepare(self, entries: list[StepEntry]) -> PreparedStep:
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


class DecodeGraph:
    """One captured CUDA graph of the model's forward pass plus sampling for a fixed number of
    single-token requests.  Its inputs live in one static int32 buffer that is refilled (one upload)
    before every replay; rows beyond the live requests are padding (context length 0, slot -1)."""

    def __init__(self, runner: "ModelRunner", batch: int, max_ctx: int, greedy: bool) -> None:
        cache, model = runner.cache, runner.model
        self.batch, self.greedy = batch, greedy
        self.max_blocks = (max_ctx + cache.page_size - 1) // cache.page_size
        G = len(cache.groups)
        seg, off = {}, 0
        # values that the parts' kernels read from device memory and that change with the live requests
        # (``Part.step_scalars``): one word each, refreshed before every replay
        self._scalar_rules = model.step_scalars()
        for name, size in (("tokens", batch), ("positions", batch), ("tok_seq", batch), ("q_start", batch + 1),
                           ("ctx_lens", batch), ("rows", batch), ("temperature", batch), ("top_k", batch),
                           ("top_p", batch), ("uniform", batch), *((f"scalar:{name}", 1) for name in self._scalar_rules)):
            seg[name] = (off, size)
            off += _pad4(size)
        for g in range(G):
            seg[f"slots{g}"] = (off, batch)
            off += _pad4(batch)
            seg[f"tables{g}"] = (off, batch * self.max_blocks)
            off += _pad4(batch * self.max_blocks)
        self.seg, self.size = seg, off
        self.host = torch.zeros(off, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(off, dtype=torch.int32, device=runner.device)
        h = self.host.numpy()
        self.h = {name: h[o : o + n] for name, (o, n) in seg.items()}
        self.hf = {name: h[o : o + n].view(np.float32) for name, (o, n) in seg.items()
                   if name in ("temperature", "top_p", "uniform")}
        for g in range(G):
            self.h[f"tables{g}"] = self.h[f"tables{g}"].reshape(batch, self.max_blocks)
        self.h["q_start"][:] = np.arange(batch + 1)
        self.h["rows"][:] = np.arange(batch)
        self.upload_bytes = off * 4
        self._uploaded = torch.cuda.Event()
        # which request's table each row holds and how much of it, so that a step writes only the
        # pages a request gained since its last step
        self._row_owner: list[list] = [[None] * batch for _ in range(G)]  # per group and row: (request, table length held, its table_epoch)

        def view(name):
            o, n = seg[name]
            return self.dev[o : o + n]

        ctx = StepContext(
            dtype=model.dtype, device=runner.device, status=runner.status, num_tokens=batch, num_seqs=batch,
            positions=view("positions"), tok_seq=view("tok_seq"), q_start=view("q_start"), ctx_lens=view("ctx_lens"),
            q_lens_host=[1] * batch, ctx_lens_host=[max_ctx] * batch, max_q_len=1, max_ctx_len=max_ctx,
        )
        ctx.views = cache.views([view(f"tables{g}").view(batch, self.max_blocks) for g in range(G)],
                                [view(f"slots{g}") for g in range(G)], None, [])
        for name, rule in self._scalar_rules.items():
            ctx.extras[name] = view(f"scalar:{name}")
            self.h[f"scalar:{name}"][0] = rule(batch, max_ctx)

        def run():
            # the logits of every row stay readable after a replay (trace replay reads them; generation
            # reads the sampled tokens only)
            logits = self.logits = model.forward(ctx, view("tokens"), view("rows"))
            if greedy:
                return ops.argmax(logits)
            return ops.sample(logits, view("temperature").view(torch.float32), view("top_k"),
                              view("top_p").view(torch.float32), view("uniform").view(torch.float32))

        self._fill_padding(0)
        self.dev.copy_(self.host)
        before = launch_count()
        run()  # eager warm-up: scratch buffers and kernel attributes are set up outside the capture
        self.kernels = launch_count() - before
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = run()
        torch.cuda.synchronize()

    def _fill_padding(self, live: int) -> None:
        h = self.h
        h["tokens"][live:] = 0
        h["positions"][live:] = 0
        h["tok_seq"][live:] = -1
        h["ctx_lens"][live:] = 0
        for name in h:
            if name.startswith("slots"):
                h[name][live:] = -1

    def replay(self, cache: CacheManager, reqs, tokens: list[int], sampling=None) -> torch.Tensor:
        """Refill the inputs for these requests (each brings one token, its slot already
        reserved), upload them in one copy, replay.  ``sampling``: (temperature, top_k, top_p,
        uniform) lists for a graph that samples.  Returns the sampled tokens of the live rows."""
        self.fill(cache, reqs, sampling)
        return self.launch(tokens)

    def fill(self, cache: CacheManager, reqs, sampling=None) -> None:
        """Everything of a step's inputs but the token ids, written into the pinned buffer: it depends
        on the requests' positions and pages only, so it can be done while the step before is still
        running (its upload has long left the buffer)."""
        n = self._filled = len(reqs)
        self._uploaded.synchronize()  # the last upload has left the pinned buffer
        h, ps = self.h, cache.page_size
        pos = np.fromiter((r.num_computed for r in reqs), dtype=np.int32, count=n)
        h["positions"][:n] = pos
        h["tok_seq"][:n] = np.arange(n, dtype=np.int32)
        h["ctx_lens"][:n] = pos + 1
        rows = np.arange(n)
        for g in range(len(cache.groups)):
            tables, slots = h[f"tables{g}"], h[f"slots{g}"]
            owners = self._row_owner[g]
            for i, r in enumerate(reqs):
                # a row is rewritten only from where the request's table grew since the row last held it
                # (most steps: nowhere)
                table = r.tables[g]
                owner = owners[i]
                if owner is not None and owner[0] is r and owner[1] == len(table) and owner[2] == r.table_epoch:
                    continue
                same = owner is not None and owner[0] is r and owner[2] == r.table_epoch and owner[1] <= len(table)
                have = owner[1] if same else 0
                tables[i, have : len(table)] = table[have:]
                owners[i] = (r, len(table), r.table_epoch)
            pages = tables[rows, pos // ps]
            if (pages == NO_PAGE).any():
                bad = reqs[int(np.argmax(pages == NO_PAGE))]
                raise RuntimeError(f"request {bad.request_id!r}: a token lands in a page that was given back")
            slots[:n] = pages * ps + pos % ps
        if sampling is not None:
            temperature, top_k, top_p, uniform = sampling
            self.hf["temperature"][:n] = temperature
            h["top_k"][:n] = top_k
            self.hf["top_p"][:n] = top_p
            self.hf["uniform"][:n] = uniform
            self.hf["temperature"][n:] = 0.0
        self._fill_padding(n)
        longest = int(pos.max()) + 1
        for name, rule in self._scalar_rules.items():
            h[f"scalar:{name}"][0] = rule(n, longest)

    def launch(self, tokens: list[int]) -> torch.Tensor:
        """The token ids of the filled step, one upload, the replay.  Returns the sampled tokens."""
        n = self._filled
        self.h["tokens"][:n] = tokens
        self.dev.copy_(self.host, non_blocking=True)
        self._uploaded.record()
        self.graph.replay()
        return self.out[:n]


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
        self.graph_max_batch = 0
        self.graph_kernel_launches = 0  # kernels replayed through graphs (for accounting)
        self.last_graph: DecodeGraph | None = None  # the graph of the last captured step that ran
        self.last_upload_bytes = 0

    def enable_graphs(self, max_ctx: int, max_batch: int) -> bool:
        """Let steps in which every request brings exactly one token replay a captured CUDA graph
        (one per batch-size bucket).  Only for models whose parts are all safe to capture."""
        if not self.model.graph_safe() or self.cache.state.needs:
            return False
        self.graph_max_ctx, self.graph_max_batch = max_ctx, max_batch
        self.model.reserve_for_steps(max_batch, max_ctx)  # scratch that captured graphs point at is set up once
        return True

    def can_use_graph(self, entries: list[StepEntry]) -> bool:
        return (self.graph_max_batch > 0 and 0 < len(entries) <= self.graph_max_batch
                and all(len(e.tokens) == 1 for e in entries))

    def decode_with_graph(self, entries: list[StepEntry], sampling=None) -> torch.Tensor:
        """One single-token step for every entry through the captured graph, sampling included.
        Returns the sampled tokens (device int32 [len(entries)])."""
        prepared = self.prepare_decode([e.request_id for e in entries], sampling)
        return self.launch_decode(prepared, [e.tokens[0] for e in entries])

    def prepare_decode(self, request_ids: list[str], sampling=None):
        """The first half of ``decode_with_graph``: slots reserved, graph chosen, every input but the
        token ids written.  It needs the requests' positions only, so the engine may call it for step
        N+1 while step N runs (after step N's launch: positions are advanced at launch)."""
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
        key = (bucket, sampling is None, tier)
        graph = self.graphs.get(key)
        if graph is None:
            graph = self.graphs[key] = DecodeGraph(self, bucket, tier, greedy=sampling is None)
        graph.fill(cache, reqs, sampling)
        return graph, reqs

    def launch_decode(self, prepared, tokens: list[int]) -> torch.Tensor:
        """The second half: the token ids, the upload, the replay; positions advance."""
        graph, reqs = prepared
        cache = self.cache
        out = graph.launch(tokens)
        self.last_graph = graph
        self.graph_kernel_launches += graph.kernels
        self.last_upload_bytes = graph.upload_bytes
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
        prepared = self.builder.prepare(entries)
        logits = self.model.forward(prepared.ctx, prepared.token_ids, prepared.logit_rows)
        self.builder.commit(prepared)
        self.last_upload_bytes = self.builder.last_upload_bytes
        self.steps_run += 1
        return logits

    def check_status(self) -> None:
        """Raise if any kernel of a step reported since the last check: an index out of range (which
        it skipped) or a device-side wait that gave up.  The step's kernels, the tensor-core products
        included, all report into the device's one status word (``ops.device_status``)."""
        ops.raise_on_status(self.status)
