"""The synchronous engine: requests in, tokens out.

API after the reference's ``clockwork/engine/llm_engine.py:35-177``: ``add_request``, ``step``,
``generate``, ``abort_request``, ``has_unfinished_requests``, ``stats``.  One ``step`` is: schedule,
run the scheduled portions as one batch through the step function, sample where a sequence's
last token was computed, record prompt pages in the prefix cache, detect finished sequences,
free them (``llm_engine.py:99-125``).  Finish rules are the reference's (``:200-242``): an EOS
token (unless ``ignore_eos``) or a ``stop_token_ids`` token ends with "stop" and stays in the
output; stop strings end with "stop" when a tokenizer is present; ``max_tokens`` or
``max_model_len`` end with "length".

A tokenizer is optional here (the reference requires one, ``:42-43``): without it prompts are
token ids and texts stay empty.
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
from .step import ModelRunner, StepEntry


def _eos_ids(tokenizer, spec) -> frozenset[int]:
    # clockwork/engine/llm_engine.py:24-32: the tokenizer's EOS, else config.json's, else none
    eos = getattr(tokenizer, "eos_token_id", None) if tokenizer is not None else None
    if eos is None:
        return frozenset(spec.eos_token_ids)
    return frozenset({eos}) if isinstance(eos, int) else frozenset(eos)


class LLMEngine:
    def __init__(self, cfg: EngineConfig, model: DecoderModel | None = None, tokenizer=None,
                 device: str = "cuda:0") -> None:
        self.cfg = cfg
        if model is None:
            model = load_model(cfg.model.model, cfg.model.dtype, device)
        self.model = model
        self.tokenizer = tokenizer
        needs = model.cache_needs()
        slots = cfg.cache.num_state_slots or cfg.scheduler.max_num_seqs
        self.cache = CacheManager(
            needs, num_pages=cfg.cache.num_blocks, page_size=cfg.cache.block_size, dtype=model.dtype,
            device=model.device, num_state_slots=slots, watermark=cfg.cache.watermark,
        )
        # prefixes can be shared only when one group of full-attention layers holds all state
        shareable = (
            len(self.cache.groups) == 1 and self.cache.groups[0].need.window is None
            and not self.cache.state.needs
            and all(isinstance(n, PagedKVNeed) for n in needs.values())
        )
        self.prefix_cache = PrefixCache(
            self.cache.groups[0].allocator if self.cache.groups else None, cfg.cache.block_size,
            enabled=cfg.cache.enable_prefix_cache and shareable,
        ) if self.cache.groups else None
        self.scheduler = Scheduler(cfg.scheduler, self.cache, self.prefix_cache)
        self.runner = ModelRunner(model, self.cache)
        self.sampler = Sampler(model.device, default_seed=cfg.model.seed)
        self.uses_graphs = bool(cfg.model.cuda_graphs) and self.runner.enable_graphs(
            cfg.model.max_model_len, cfg.scheduler.max_num_seqs)
        self._eos = _eos_ids(tokenizer, model.spec)
        self._seqs: dict[str, Sequence] = {}
        self._texts: dict[str, str] = {}
        # arrival is a counter, not a clock, so scheduling never depends on wall time
        # (clockwork/engine/llm_engine.py:57-59)
        self._arrival = itertools.count()
        self._generate_counter = itertools.count()
        self._unchecked_steps = 0
        self._ahead = None  # (plan, sequences, prepared graph inputs) of the next step, made while a step ran
        self.plan_ahead = True  # False: every step is planned after the one before it was read back
        self.steps_planned_ahead = 0

    @classmethod
    def from_config(cls, cfg: EngineConfig) -> "LLMEngine":
        return cls(cfg)

    @classmethod
    def from_model_dir(cls, model_dir: str | Path, **overrides) -> "LLMEngine":
        return cls(EngineConfig.defaults(str(model_dir), **overrides))

    # ---- requests ---------------------------------------------------------------------------------
    def add_request(self, request_id: str, prompt: str | None = None,
                    sampling_params: SamplingParams | None = None,
                    prompt_token_ids: list[int] | None = None) -> None:
        """Queue one request; exactly one of ``prompt`` and ``prompt_token_ids``
        (clockwork/engine/llm_engine.py:67-97)."""
        if (prompt is None) == (prompt_token_ids is None):
            raise ValueError("provide exactly one of prompt or prompt_token_ids")
        if request_id in self._seqs:
            raise ValueError(f"request id {request_id!r} is already active")
        if prompt_token_ids is None:
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; pass prompt_token_ids instead")
            prompt_token_ids = self.tokenizer.encode(prompt)
        prompt_token_ids = [int(t) for t in prompt_token_ids]
        if not prompt_token_ids:
            raise ValueError("prompt must contain at least one token")
        if len(prompt_token_ids) >= self.cfg.model.max_model_len:
            raise ValueError(
                f"prompt of {len(prompt_token_ids)} tokens leaves no room to generate "
                f"within max_model_len {self.cfg.model.max_model_len}"
            )
        vocab = self.model.spec.vocab_size
        bad = [t for t in prompt_token_ids if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"prompt holds token ids outside the vocabulary of {vocab}: {bad[:5]}")
        params = sampling_params if sampling_params is not None else SamplingParams()
        if params.stop and self.tokenizer is None:
            raise ValueError("stop strings need a tokenizer; use stop_token_ids")
        seq = Sequence(request_id, prompt_token_ids, params, arrival_time=float(next(self._arrival)))
        self._seqs[request_id] = seq
        self._texts[request_id] = ""
        self._ahead = None  # a plan made for the running batch alone no longer holds
        self.scheduler.add_seq(seq)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    def abort_request(self, request_id: str) -> None:
        self._ahead = None
        self.scheduler.abort(request_id)
        self._forget(request_id)

    def _forget(self, request_id: str) -> None:
        self._seqs.pop(request_id, None)
        self._texts.pop(request_id, None)

    # ---- one iteration ------------------------------------------------------------------------------
    STATUS_CHECK_EVERY = 16

    def step(self) -> list[RequestOutput]:
        ahead, self._ahead = self._ahead, None
        prepared = None
        if ahead is not None and ahead[3] != self.runner.steps_run:
            ahead = None  # somebody has stepped the runner directly in between: the plan's positions are stale
        if ahead is not None:
            # planned and prepared while the last step ran: every running sequence decodes one token
            out, sampled_seqs, prepared, _ = ahead
            self.scheduler.accept_plan(out)
            self.steps_planned_ahead += 1
            entries = None
        else:
            out = self.scheduler.schedule()
            if not out.portions:
                if out.preempted or not self.scheduler.has_unfinished():
                    return []
                # admission stalled with nothing running: pages held only by the prefix cache are
                # invisible to the scheduler; reclaim the idle ones and retry once
                # (clockwork/engine/llm_engine.py:102-113)
                if self.prefix_cache is not None and self.prefix_cache.evict(self.cache.num_pages) > 0:
                    out = self.scheduler.schedule()
                if not out.portions:
                    raise RuntimeError("waiting request cannot be admitted even with an empty prefix cache")
            entries = []
            sampled_seqs = []
            for p in out.portions:
                tokens = p.seq.tokens_between(p.start, p.start + p.num_tokens)
                entries.append(StepEntry(p.seq.seq_id, tokens, [p.num_tokens - 1] if p.samples else []))
                if p.samples:
                    sampled_seqs.append(p.seq)
        tokens: list[int] = []
        if prepared is not None or (len(sampled_seqs) == len(entries) and self.runner.can_use_graph(entries)):
            # every request decodes one token: replay the captured graph (forward pass + sampling)
            if prepared is None:
                sampling = self.sampler.host_params(
                    [s.sampling_params for s in sampled_seqs], [len(s.output_token_ids) for s in sampled_seqs])
                prepared = self.runner.prepare_decode([e.request_id for e in entries], sampling)
                fed = [e.tokens[0] for e in entries]
            else:
                fed = [s.output_token_ids[-1] for s in sampled_seqs]
            device_tokens = self.runner.launch_decode(prepared, fed)
            # While the GPU runs this step, the host plans and prepares the next one on the assumption
            # that every sequence goes on (dropped below if one ends, and whenever a request arrives or
            # is aborted): the GPU then does not wait for the scheduler and the step builder.
            self._ahead = self._plan_ahead() if self.plan_ahead else None
            tokens = device_tokens.tolist()
            self._unchecked_steps += 1
        else:
            logits = self.runner.step(entries)
            if sampled_seqs:
                tokens = self.sampler.sample(
                    logits, [s.sampling_params for s in sampled_seqs], [len(s.output_token_ids) for s in sampled_seqs]
                )
            self._unchecked_steps = self.STATUS_CHECK_EVERY  # steps with prompt portions are checked at once
        # The kernels' status words cost a device-to-host read of their own: after a captured decode step
        # they are read every STATUS_CHECK_EVERY steps (a kernel that met an index out of range has skipped
        # the access and goes on reporting; the error is raised a few steps late, never lost).
        if self._unchecked_steps >= self.STATUS_CHECK_EVERY:
            self.runner.check_status()
            self._unchecked_steps = 0
        for p in out.portions:
            p.seq.num_computed_tokens = p.start + p.num_tokens
        for seq, token in zip(sampled_seqs, tokens):
            seq.append_token(int(token))
        if self.prefix_cache is not None and self.prefix_cache.enabled:
            for seq in out.prefill_seqs:
                # whole pages of the prompt that are computed by now
                # (clockwork/engine/llm_engine.py:115-119 inserts after every prefill)
                n = min(seq.num_computed_tokens, len(seq.prompt_token_ids))
                req = self.cache.requests.get(seq.seq_id)
                if req is not None and n >= self.cache.page_size:
                    self.prefix_cache.insert(seq.prompt_token_ids[:n], req.tables[0])
        outputs = [self._process(seq) for seq in sampled_seqs]
        finished = [output for output in outputs if output.finished]
        if finished:
            self.scheduler.free_finished()
            for output in finished:
                self._forget(output.request_id)
            self._ahead = None  # the plan assumed that every sequence goes on
            if self._unchecked_steps:
                self.runner.check_status()  # no request ends with an unread status
                self._unchecked_steps = 0
        return outputs

    def _plan_ahead(self):
        """The next step's plan and graph inputs, if the next step can be foreseen (see ``step``)."""
        out = self.scheduler.plan_next_decode(self.cfg.model.max_model_len)
        if out is None:
            return None
        seqs = [p.seq for p in out.portions]
        if not 0 < len(seqs) <= self.runner.graph_max_batch:
            return None
        sampling = self.sampler.host_params([s.sampling_params for s in seqs], [len(s.output_token_ids) + 1 for s in seqs])
        # (the runner's step count says at the next step whether anybody else has stepped it since)
        return out, seqs, self.runner.prepare_decode([s.seq_id for s in seqs], sampling), self.runner.steps_run

    def _finish_rules(self, seq: Sequence) -> None:
        """The request's finish rules in the form the per-step check wants them."""
        params = seq.sampling_params
        stops = set(params.stop_token_ids)
        if not params.ignore_eos:
            stops |= set(self._eos)
        seq.stop_ids = frozenset(stops) if stops else None
        seq.length_limit = min(params.max_tokens, self.cfg.model.max_model_len - len(seq.prompt_token_ids))

    def _process(self, seq: Sequence) -> RequestOutput:
        if seq.length_limit is None:
            self._finish_rules(seq)
        out_ids = seq.output_token_ids
        n_out = len(out_ids)
        stops = seq.stop_ids
        if self.tokenizer is None:
            # the usual case on this path: token rules only, one object per request and step
            if stops is not None and out_ids[-1] in stops:
                seq.status = SequenceStatus.FINISHED_STOPPED
                return RequestOutput(seq, n_out, True, "stop")
            if n_out >= seq.length_limit:
                seq.status = SequenceStatus.FINISHED_LENGTH
                return RequestOutput(seq, n_out, True, "length")
            return RequestOutput(seq, n_out, False, None)
        params = seq.sampling_params
        finish_reason = None
        delta = ""
        text = self._texts.get(seq.seq_id, "")
        if stops is not None and out_ids[-1] in stops:
            finish_reason = "stop"  # the stopping token stays in token_ids, adds no text
        else:
            candidate = self.tokenizer.decode(out_ids)
            if params.stop:
                hits = [pos for pos in (candidate.find(s) for s in params.stop) if pos >= 0]
                if hits:
                    candidate = candidate[: min(hits)]
                    finish_reason = "stop"
            delta = candidate[len(text):] if candidate.startswith(text) else ""
            text = candidate
            self._texts[seq.seq_id] = text
        if finish_reason is None and n_out >= seq.length_limit:
            finish_reason = "length"
        if finish_reason == "stop":
            seq.status = SequenceStatus.FINISHED_STOPPED
        elif finish_reason == "length":
            seq.status = SequenceStatus.FINISHED_LENGTH
        return RequestOutput(seq, n_out, finish_reason is not None, finish_reason, text, delta)

    # ---- whole requests -------------------------------------------------------------------------------
    def generate(self, prompts: list[str] | list[list[int]],
                 sampling_params: SamplingParams | list[SamplingParams] | None = None) -> list[RequestOutput]:
        """Run prompts to completion; final outputs in prompt order
        (clockwork/engine/llm_engine.py:135-159)."""
        ids: list[str] = []
        for i, prompt in enumerate(prompts):
            rid = f"generate-{next(self._generate_counter)}"
            ids.append(rid)
            params = sampling_params[i] if isinstance(sampling_params, list) else sampling_params
            if isinstance(prompt, str):
                self.add_request(rid, prompt=prompt, sampling_params=params)
            else:
                self.add_request(rid, prompt_token_ids=prompt, sampling_params=params)
        finals: dict[str, RequestOutput] = {}
        pending = set(ids)
        while pending:
            outputs = self.step()
            for output in outputs:
                if output.finished and output.request_id in pending:
                    finals[output.request_id] = output
                    pending.discard(output.request_id)
            if not outputs and not self.scheduler.has_unfinished():
                raise RuntimeError(f"engine drained with unfinished requests: {sorted(pending)}")
        return [finals[rid] for rid in ids]

    def decode_step_device(self, request_ids: list[str], tokens: list[list[int]]) -> torch.Tensor:
        """One step for requests that are already in the cache, with the given next tokens, sampled
        greedily on the device and not read back: the step function and sampler without the
        scheduler's bookkeeping (used to time the device work alone)."""
        from .. import ops

        self._ahead = None
        entries = [StepEntry(rid, toks, [len(toks) - 1]) for rid, toks in zip(request_ids, tokens)]
        if self.runner.can_use_graph(entries):
            return self.runner.decode_with_graph(entries, None)
        return ops.argmax(self.runner.step(entries))

    def stats(self) -> dict:
        sched = self.scheduler.stats
        out = {
            "num_waiting": sched.num_waiting,
            "num_running": sched.num_running,
            "num_preempted_total": sched.num_preempted_total,
            "num_scheduled_batches": sched.num_scheduled_batches,
            "total_prompt_tokens": sched.total_prompt_tokens,
            "total_cached_tokens": sched.total_cached_tokens,
            "num_free_blocks": min(self.cache.num_free_pages()) if self.cache.groups else 0,
        }
        if self.prefix_cache is not None:
            cache = self.prefix_cache.stats
            out.update(prefix_cache_queries=cache.queries, prefix_cache_hit_tokens=cache.hit_tokens,
                       prefix_cache_prompt_tokens=cache.prompt_tokens, prefix_cache_hit_rate=cache.hit_rate)
        return out
