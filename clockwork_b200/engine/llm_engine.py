"""The synchronous engine: requests in, tokens out.

The calls are the reference's (``clockwork/engine/llm_engine.py:35-177``): ``add_request``, ``step``,
``generate``, ``abort_request``, ``has_unfinished_requests``, ``stats``; a tokenizer is optional here
(the reference requires one, ``:42-43``): without it prompts are token ids and texts stay empty.  A
step is: schedule; run the scheduled portions as one batch through the step function; sample where a
request's last token was computed; record whole prompt pages in the prefix cache; see which requests
have ended; give their memory back (``:99-125``).  A request ends as in the reference (``:200-242``): a
stop token (EOS unless ``ignore_eos``, or one of ``stop_token_ids``) ends it with "stop" and stays in
the output, a stop string ends it with "stop" when there is a tokenizer, ``max_tokens`` or
``max_model_len`` end it with "length".

What is different is how steps in which every running request decodes one token are run.  Their
inputs come from the per-request state table on the device (``cache.state.request``), which the
sampling kernel of the step before has already updated, so such a step is launched *before* the
tokens of the step before it have been read: while the GPU runs step N+1, the host reads step N's
tokens, appends them, and sees who has ended.  A request that turns out to have ended in step N has
then computed one token too many; that token is thrown away (its page was the request's own and goes
back with the others).  Steps that admit, preempt or run prompt portions go the plain way: they are
planned after everything before them has been read.
"""

from __future__ import annotations

import itertools
from pathlib import Path

import torch

from ..cache.manager import CacheManager
from ..cache.prefix import PrefixCache
from ..config.engine import EngineConfig
from ..parts.base import PagedKVNeed
from ..parts.model import DecoderModel
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model
from .scheduler import Scheduler
from .sequence import RequestOutput, Sequence, SequenceStatus
from .step import ModelRunner, StepEntry, fresh_row
from .. import ops


class _Launched:
    """A captured single-token step that has been launched and whose tokens have not been read yet."""

    __slots__ = ("seqs", "portions", "tokens", "arrived")

    def __init__(self, seqs, portions, tokens: torch.Tensor, arrived: torch.cuda.Event) -> None:
        self.seqs = seqs          # the sequences of the step's rows
        self.portions = portions  # the plan's portions, in the same order
        self.tokens = tokens      # pinned int32 [rows + status words]: sampled tokens, then the kernels' status
        self.arrived = arrived    # recorded after the copy of `tokens`


class LLMEngine:
    STATUS_WORDS = 4

    def __init__(self, cfg: EngineConfig, model: DecoderModel | None = None, tokenizer=None,
                 device: str = "cuda:0") -> None:
        self.cfg = cfg
        self.model = model if model is not None else load_model(cfg.model.model, cfg.model.dtype, device)
        self.tokenizer = tokenizer
        model = self.model
        needs = model.cache_needs()
        self.cache = CacheManager(
            needs, num_pages=cfg.cache.num_blocks, page_size=cfg.cache.block_size, dtype=model.dtype, device=model.device,
            num_state_slots=cfg.cache.num_state_slots or cfg.scheduler.max_num_seqs, watermark=cfg.cache.watermark,
        )
        self.prefix_cache = None
        if self.cache.groups:
            # prefixes can be shared by pages only when pages are all a request keeps: one group of layers
            # that keep every key, and no mixer with state of its own
            pages_only = (len(self.cache.groups) == 1 and self.cache.groups[0].need.window is None
                          and not self.cache.state.needs and all(isinstance(n, PagedKVNeed) for n in needs.values()))
            self.prefix_cache = PrefixCache(self.cache.groups[0].allocator, cfg.cache.block_size,
                                            enabled=cfg.cache.enable_prefix_cache and pages_only)
        self.scheduler = Scheduler(cfg.scheduler, self.cache, self.prefix_cache)
        self.runner = ModelRunner(model, self.cache)
        self.sampler = Sampler(model.device, default_seed=cfg.model.seed)
        self.uses_graphs = bool(cfg.model.cuda_graphs) and self.runner.enable_graphs(
            cfg.model.max_model_len, cfg.scheduler.max_num_seqs)
        self._eos = self._end_of_sequence_ids()
        self._seqs: dict[str, Sequence] = {}
        self._texts: dict[str, str] = {}
        # arrival is a counter, not a clock: the schedule never depends on wall time
        # (clockwork/engine/llm_engine.py:57-59)
        self._ticket = itertools.count()
        self._generate_calls = itertools.count()
        self._launched: _Launched | None = None  # the step whose tokens the next call of ``step`` reads
        self.run_ahead = True  # False: no step is launched before the one before it has been read
        self.steps_run_ahead = 0
        rows = max(1, cfg.scheduler.max_num_seqs) + self.STATUS_WORDS
        self._landing = [torch.zeros(rows, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._landing_turn = 0

    @classmethod
    def from_config(cls, cfg: EngineConfig) -> "LLMEngine":
        return cls(cfg)

    @classmethod
    def from_model_dir(cls, model_dir: str | Path, **overrides) -> "LLMEngine":
        return cls(EngineConfig.defaults(str(model_dir), **overrides))

    def _end_of_sequence_ids(self) -> frozenset[int]:
        """The tokenizer's end-of-sequence id(s) when it has any, else config.json's, else none
        (clockwork/engine/llm_engine.py:24-32)."""
        named = getattr(self.tokenizer, "eos_token_id", None)
        if named is None:
            named = self.model.spec.eos_token_ids
        return frozenset([named] if isinstance(named, int) else named or ())

    # ---- requests ---------------------------------------------------------------------------------
    def add_request(self, request_id: str, prompt: str | None = None,
                    sampling_params: SamplingParams | None = None,
                    prompt_token_ids: list[int] | None = None) -> None:
        """Queue one request, given either as text (needs a tokenizer) or as token ids
        (clockwork/engine/llm_engine.py:67-97)."""
        if request_id in self._seqs:
            raise ValueError(f"request id {request_id!r} is already active")
        given = [x for x in (prompt, prompt_token_ids) if x is not None]
        if len(given) != 1:
            raise ValueError("a request is exactly one of prompt (text) or prompt_token_ids")
        if prompt_token_ids is None:
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; pass prompt_token_ids instead")
            prompt_token_ids = self.tokenizer.encode(prompt)
        ids = [int(t) for t in prompt_token_ids]
        limit, vocab = self.cfg.model.max_model_len, self.model.spec.vocab_size
        if not ids:
            raise ValueError("a prompt must hold at least one token")
        if len(ids) >= limit:
            raise ValueError(f"a prompt of {len(ids)} tokens leaves no room to generate: max_model_len is {limit}")
        strays = [t for t in ids if not 0 <= t < vocab]
        if strays:
            raise ValueError(f"token ids outside the vocabulary of {vocab}: {strays[:5]}")
        params = sampling_params or SamplingParams()
        if params.stop and self.tokenizer is None:
            raise ValueError("stop strings need a tokenizer; use stop_token_ids")
        seq = Sequence(request_id, ids, params, arrival_time=float(next(self._ticket)))
        ends = set(params.stop_token_ids) | (set() if params.ignore_eos else self._eos)
        seq.stop_ids = frozenset(ends) or None
        seq.length_limit = min(params.max_tokens, limit - len(ids))
        self._seqs[request_id] = seq
        self._texts[request_id] = ""
        self.scheduler.add_seq(seq)

    def capture_graphs_ahead(self, decode_batches=(1, 8), prompt_tokens=(128, 512, 2048), max_ctx: int = 1024,
                             greedy: bool = True) -> int:
        """Captures the CUDA graphs of the usual steps now instead of at their first use (see
        ``ModelRunner.capture_ahead``).  Returns how many were captured; 0 when graphs are off."""
        if not self.uses_graphs:
            return 0
        return self.runner.capture_ahead(decode_batches, prompt_tokens, max_ctx, greedy)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    def abort_request(self, request_id: str) -> None:
        """(A step that is already running with this request finishes; its token for it is dropped.)"""
        self.scheduler.abort(request_id)
        self._forget(request_id)

    def _forget(self, request_id: str) -> None:
        self._seqs.pop(request_id, None)
        self._texts.pop(request_id, None)

    # ---- one iteration ------------------------------------------------------------------------------
    def step(self) -> list[RequestOutput]:
        launched, self._launched = self._launched, None
        if launched is not None:
            return self._read(launched)
        plan = self.scheduler.schedule()
        if not plan.portions:
            if plan.preempted or not self.scheduler.has_unfinished():
                return []
            # nothing runs and nothing could be admitted: pages that only the prefix cache still holds
            # are not free; let it give the idle ones back and try once more
            # (clockwork/engine/llm_engine.py:102-113)
            if self.prefix_cache is not None and self.prefix_cache.evict(self.cache.num_pages) > 0:
                plan = self.scheduler.schedule()
            if not plan.portions:
                raise RuntimeError("waiting request cannot be admitted even with an empty prefix cache")
        entries = [StepEntry(p.seq.seq_id, p.seq.tokens_between(p.start, p.start + p.num_tokens),
                             [p.num_tokens - 1] if p.samples else []) for p in plan.portions]
        sampled = [p.seq for p in plan.portions if p.samples]
        if len(sampled) == len(entries) and self.runner.can_use_graph(entries):
            # every request decodes one token: the captured step, its inputs set from what the host knows
            return self._read(self._launch(plan.portions, fresh=True))
        logits = self.runner.step(entries)
        tokens: list[int] = []
        if sampled:
            tokens = self.sampler.sample(logits, [s.sampling_params for s in sampled], [len(s.output_token_ids) for s in sampled])
        self.runner.check_status()
        for p in plan.portions:
            p.seq.num_computed_tokens = p.start + p.num_tokens
        if self.prefix_cache is not None and self.prefix_cache.enabled:
            for seq in plan.prefill_seqs:
                # whole pages of the prompt that are computed by now
                # (clockwork/engine/llm_engine.py:115-119 inserts after every prefill)
                n = min(seq.num_computed_tokens, len(seq.prompt_token_ids))
                req = self.cache.requests.get(seq.seq_id)
                if req is not None and n >= self.cache.page_size:
                    self.prefix_cache.insert(seq.prompt_token_ids[:n], req.tables[0])
        return self._outputs(sampled, tokens)

    def _launch(self, portions, fresh: bool) -> _Launched:
        """Launch a captured single-token step for the portions' sequences and start the copy of its
        tokens (and of the kernels' status words) to the host.  ``fresh``: the requests' device state is
        set from what the host knows (their last tokens have been read); otherwise it goes on from what
        the step before left on the device."""
        seqs = [p.seq for p in portions]
        rows = None
        sampling = self.sampler.state_rows([s.sampling_params for s in seqs], [len(s.output_token_ids) for s in seqs])
        if fresh:
            rows = []
            for i, (p, seq) in enumerate(zip(portions, seqs)):
                last = seq.tokens_between(p.start, p.start + 1)[0]  # the token this step feeds
                if sampling is None:
                    rows.append(fresh_row(p.start, last))
                else:
                    temperature, top_k, top_p, seed, draws = sampling[i]
                    rows.append(fresh_row(p.start, last, draws, seed, temperature, top_k, top_p))
        prepared = self.runner.prepare_decode([s.seq_id for s in seqs], rows, greedy=sampling is None)
        device_tokens = self.runner.launch_decode(prepared)
        n = len(seqs)
        landing = self._landing[self._landing_turn]
        self._landing_turn = (self._landing_turn + 1) % len(self._landing)
        landing[:n].copy_(device_tokens, non_blocking=True)
        landing[n : n + self.STATUS_WORDS].copy_(self.runner.status, non_blocking=True)
        arrived = torch.cuda.Event()
        arrived.record()
        return _Launched(seqs, portions, landing, arrived)

    def _read(self, launched: _Launched) -> list[RequestOutput]:
        """Read a launched step's tokens.  Before waiting for them, launch the step after it if it can be
        foreseen: every sequence of this step is still wanted, nothing waits, nobody ends by length."""
        live = [not s.status.finished for s in launched.seqs]
        if self.run_ahead and all(live):
            plan = self.scheduler.plan_next_decode(self.cfg.model.max_model_len)
            if plan is not None and 0 < len(plan.portions) <= self.runner.graph_max_batch and self.uses_graphs:
                self.scheduler.accept_plan(plan)
                self._launched = self._launch(plan.portions, fresh=False)
                self.steps_run_ahead += 1
        launched.arrived.synchronize()
        n = len(launched.seqs)
        words = launched.tokens[: n + self.STATUS_WORDS].tolist()
        if words[n] != 0:
            self.runner.check_status()  # raises with the kernels' report
        sampled, tokens = [], []
        for seq, portion, token, alive in zip(launched.seqs, launched.portions, words, live):
            if alive:  # (a sequence that ended or was aborted while this step ran: its token is dropped)
                seq.num_computed_tokens = portion.start + portion.num_tokens
                sampled.append(seq)
                tokens.append(token)
        return self._outputs(sampled, tokens)

    def _outputs(self, sampled: list[Sequence], tokens: list[int]) -> list[RequestOutput]:
        outputs = []
        ended = False
        for seq, token in zip(sampled, tokens):
            seq.append_token(int(token))
            out = self._judge(seq)
            ended = ended or out.finished
            outputs.append(out)
        if ended:
            self.scheduler.free_finished()
            for out in outputs:
                if out.finished:
                    self._forget(out.request_id)
        return outputs

    def _judge(self, seq: Sequence) -> RequestOutput:
        """Whether the token just appended ends the request, and what to report for it."""
        generated = seq.output_token_ids
        count = len(generated)
        stopped = seq.stop_ids is not None and generated[-1] in seq.stop_ids
        text = delta = ""
        if self.tokenizer is not None:
            text = self._texts.get(seq.seq_id, "")
            if not stopped:  # a stop token stays in token_ids and adds no text
                shown = self.tokenizer.decode(generated)
                cuts = [at for at in map(shown.find, seq.sampling_params.stop) if at >= 0]
                if cuts:
                    shown, stopped = shown[: min(cuts)], True
                delta = shown[len(text):] if shown.startswith(text) else ""
                text = self._texts[seq.seq_id] = shown
        if stopped:
            seq.status = SequenceStatus.FINISHED_STOPPED
        elif count >= seq.length_limit:
            seq.status = SequenceStatus.FINISHED_LENGTH
        return RequestOutput(seq, count, seq.status.finished, seq.status.finish_reason, text, delta)

    # ---- whole requests -------------------------------------------------------------------------------
    def generate(self, prompts: list[str] | list[list[int]],
                 sampling_params: SamplingParams | list[SamplingParams] | None = None) -> list[RequestOutput]:
        """Run the prompts until each has ended and return their last outputs in the prompts' order
        (clockwork/engine/llm_engine.py:135-159)."""
        per_prompt = sampling_params if isinstance(sampling_params, list) else [sampling_params] * len(prompts)
        names = [f"generate-{next(self._generate_calls)}" for _ in prompts]
        for name, prompt, params in zip(names, prompts, per_prompt):
            kind = "prompt" if isinstance(prompt, str) else "prompt_token_ids"
            self.add_request(name, sampling_params=params, **{kind: prompt})
        last: dict[str, RequestOutput] = {}
        while len(last) < len(names):
            produced = self.step()
            last.update((out.request_id, out) for out in produced if out.finished and out.request_id in names)
            if not produced and self._launched is None and not self.scheduler.has_unfinished():
                missing = sorted(set(names) - set(last))
                raise RuntimeError(f"the engine ran dry with requests unfinished: {missing}")
        return [last[name] for name in names]

    def decode_step_device(self, request_ids: list[str], tokens: list[list[int]]) -> torch.Tensor:
        """One step for requests that are already in the cache, with the given next tokens, sampled
        greedily on the device and not read back: the step function and sampler without the
        scheduler's bookkeeping (used to time the device work alone)."""
        self._launched = None
        entries = [StepEntry(rid, toks, [len(toks) - 1]) for rid, toks in zip(request_ids, tokens)]
        if self.runner.can_use_graph(entries):
            return self.runner.decode_with_graph(entries, None)
        return ops.argmax(self.runner.step(entries))

    def stats(self) -> dict:
        report = dict(vars(self.scheduler.stats))
        report["num_free_blocks"] = min(self.cache.num_free_pages(), default=0)
        if self.prefix_cache is not None:
            seen = self.prefix_cache.stats
            report.update(prefix_cache_queries=seen.queries, prefix_cache_hit_tokens=seen.hit_tokens,
                          prefix_cache_prompt_tokens=seen.prompt_tokens, prefix_cache_hit_rate=seen.hit_rate)
        return report
